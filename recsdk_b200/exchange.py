"""Sharded lookups over the GPUs of one box through the device-driven dedup exchange (`recsdk_xchg_*`).

Two placements of the rows, one machinery:

  table-wise  whole tables on ranks (the reference's TW sharding,
              hybrid_torchrec/hybrid_torchrec/distributed/sharding/hybrid_tw_sharding.py:43-82)
  row-wise    row ``id`` of every table on rank ``id % W`` at local row ``id // W``
              (hybrid_torchrec/src/ids_process/bucketize.cpp:44-48, sharding/hybrid_rw_sharding.py)

Each rank keeps one flat table with the rows it owns and, for the other ranks to write into, an inbox: per source
rank the local row numbers it asks for, their count, and one summed gradient row per asked row.  A step is three
library calls and two fences, with no host read, no allocation and no split-size collective:

    out = x.forward(indices, offsets)      # dedup, ids+count -> owners' inboxes, rows pulled from owners, pooled
    x.backward_local(grad)                 # per-row sums -> owners' gradient inboxes
    x.fence()                              # every rank's stores have landed
    x.backward_owner()                     # merge in source-rank order, optimizer once per row
    x.fence()                              # tables are final before the next forward reads them

What the reference does with all-to-alls around the lookup (ids out, rows back, gradients out; on its own hardware
the fused collectives GatherAll and AllUss, cust_op/ascendc_op/ai_core_op/lccl/v220/op_kernel/gather_all.h,
all2all_uss.h:319-381) happens inside these kernels over peer mappings.  `connect_processes` maps the buffers of
one-process-per-GPU ranks into each other with CUDA IPC; `connect_local` wires several logical ranks that live in
ONE process (one GPU or several) with plain pointers -- the same kernels, used by the single-GPU parity tests.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from . import _lib
from .ops import _stream, check, new_status, raise_on_status
from .tbe import EmbOptimType, PoolingMode

_OPT_CODE = {EmbOptimType.EXACT_ADAGRAD: _lib.OPT_ADAGRAD, EmbOptimType.ADAM: _lib.OPT_ADAM,
             EmbOptimType.EXACT_SGD: _lib.OPT_SGD}


def table_wise_layout(rows: Sequence[int], owner: Sequence[int], world: int):
    """Linear row numbering for whole tables on ranks: tables ordered by (owner, table number).
    Returns (part_base [F], rank_base [W+1])."""
    order = sorted(range(len(rows)), key=lambda f: (owner[f], f))
    base, acc = [0] * len(rows), 0
    rank_base = [0] * (world + 1)
    for f in order:
        base[f] = acc
        acc += rows[f]
        rank_base[owner[f] + 1] = acc
    for r in range(1, world + 1):
        rank_base[r] = max(rank_base[r], rank_base[r - 1])
    return base, rank_base


def row_wise_layout(rows: Sequence[int], world: int):
    """Linear row numbering for rows split by ``id % W``: rank r keeps, table after table, the rows r, r+W, ...
    Returns (part_base [W*F] indexed r*F+f, rank_base [W+1], local_rows[r][f])."""
    F = len(rows)
    local = [[max((rows[f] - r + world - 1) // world, 0) for f in range(F)] for r in range(world)]
    part_base, rank_base, acc = [0] * (world * F), [0] * (world + 1), 0
    for r in range(world):
        rank_base[r] = acc
        for f in range(F):
            part_base[r * F + f] = acc
            acc += local[r][f]
    rank_base[world] = acc
    return part_base, rank_base, local


class DedupExchange:
    """One rank's end of the exchange: its flat table (+ optimizer state), its inbox, its scratch."""

    def __init__(self, rows: Sequence[int], dim: int, world: int, rank: int, partition: str = "table",
                 owner: Optional[Sequence[int]] = None, batch_size: int = 1, max_ids: Optional[int] = None,
                 inbox_cap: Optional[int] = None, optimizer: EmbOptimType = EmbOptimType.ADAM,
                 pooling_mode: PoolingMode = PoolingMode.SUM, device="cuda", learning_rate: float = 0.01,
                 eps: float = 1e-8, beta1: float = 0.9, beta2: float = 0.999, gradient_clipping: bool = False,
                 max_gradient: float = 1.0, initial_accumulator_value: float = 0.0,
                 weights_init: Optional[tuple] = None, seed: int = 0, one_hot: bool = False,
                 double_buffer: bool = False, **_ignored):
        if not 1 <= world <= _lib.MAX_SHARDS:
            raise ValueError(f"1..{_lib.MAX_SHARDS} ranks supported")
        if dim <= 0 or dim % 4:
            raise ValueError("row width must be a positive multiple of 4")
        self.rows, self.dim, self.world, self.rank = [int(r) for r in rows], int(dim), world, rank
        self.F, self.B = len(self.rows), int(batch_size)
        self.device = torch.device(device)
        self.pooling_mode = PoolingMode(pooling_mode)
        self.optimizer = optimizer
        self.hp = dict(lr=learning_rate, eps=eps, beta1=beta1, beta2=beta2)
        self.gradient_clipping, self.max_gradient = bool(gradient_clipping), float(max_gradient)
        dev = self.device
        if partition == "table":
            if owner is None:
                raise ValueError("table-wise placement needs `owner`")
            self.owner_of = [int(o) for o in owner]
            part_base, rank_base = table_wise_layout(self.rows, self.owner_of, world)
            self.local_tables = [f for f in sorted(range(self.F), key=lambda f: (self.owner_of[f], f))
                                 if self.owner_of[f] == rank]
            self._part_code = _lib.XCHG_TABLE_WISE
            per_rank = [sum(1 for o in self.owner_of if o == r) for r in range(world)]
            default_cap_tables = max(per_rank)
        elif partition == "row":
            part_base, rank_base, self._local_rows_rf = row_wise_layout(self.rows, world)
            self.local_tables = list(range(self.F))
            self._part_code = _lib.XCHG_ROW_WISE
            default_cap_tables = self.F
        else:
            raise ValueError("partition is 'table' or 'row'")
        self.partition = partition
        self._part_base_host, self._rank_base_host = part_base, rank_base
        self.local_rows = max(rank_base[rank + 1] - rank_base[rank], 1)
        self.max_ids = int(max_ids) if max_ids is not None else self.F * self.B
        # rows one source may ask of one owner in a step: all its ids for the tables that owner can serve
        if inbox_cap is None:
            inbox_cap = -(-self.max_ids * default_cap_tables // self.F)
        self.inbox_cap = max(int(inbox_cap), 1)
        self.key_bits = max(1, int(rank_base[world]).bit_length())

        self.part_base = torch.tensor(part_base, dtype=torch.int64, device=dev)
        self.rank_base = torch.tensor(rank_base, dtype=torch.int64, device=dev)
        self.table_rows = torch.tensor(self.rows, dtype=torch.int64, device=dev)
        n = self.local_rows * self.dim
        self.weights_dev = torch.empty(n, dtype=torch.float32, device=dev)
        if weights_init is not None:
            gen = torch.Generator(device=dev)
            gen.manual_seed(seed)
            self.weights_dev.uniform_(weights_init[0], weights_init[1], generator=gen)
        else:
            self.weights_dev.zero_()
        n_state = {EmbOptimType.ADAM: 2, EmbOptimType.EXACT_ADAGRAD: 1, EmbOptimType.EXACT_SGD: 0}[optimizer]
        self.momentum1_dev = (torch.full((n,), float(initial_accumulator_value), dtype=torch.float32, device=dev)
                              if n_state >= 1 else None)
        self.momentum2_dev = torch.zeros(n, dtype=torch.float32, device=dev) if n_state >= 2 else None
        self.iter = 0
        self.inbox_ids = torch.zeros(world * self.inbox_cap, dtype=torch.int64, device=dev)
        self.inbox_counts = torch.zeros(world, dtype=torch.int64, device=dev)
        self.inbox_grads = torch.zeros(world * self.inbox_cap * self.dim, dtype=torch.float32, device=dev)
        lib = _lib.load()
        ws_bytes = lib.recsdk_xchg_workspace_bytes(self.max_ids, self.inbox_cap, world, self.dim, self.F)
        # the scratch of a step (plan, records, chunk sums, owner-side buffers).  ``double_buffer``: a second one, so
        # that the plan of the NEXT batch (plan_forward_ahead) can be made while the current step still uses its own
        self._wss = [torch.empty(ws_bytes, dtype=torch.uint8, device=dev) for _ in range(2 if double_buffer else 1)]
        self._cur = 0
        self._ws = self._wss[0]
        self._status = new_status(dev)
        self._x = _lib.XchgT()
        x = self._x
        x.world, x.rank, x.partition, x.D = world, rank, self._part_code, self.dim
        x.F, x.B, x.max_ids, x.inbox_cap, x.key_bits = self.F, self.B, self.max_ids, self.inbox_cap, self.key_bits
        # one id per bag, promised by the caller and checked on the device: the forward then stores each fetched row
        # straight to the bags that use it
        x.flags = 1 if one_hot else 0
        x.part_base, x.rank_base, x.table_rows = (self.part_base.data_ptr(), self.rank_base.data_ptr(),
                                                   self.table_rows.data_ptr())
        x.local_rows = self.local_rows
        x.workspace, x.workspace_bytes, x.dev_status = self._ws.data_ptr(), ws_bytes, self._status.data_ptr()
        self._connected = False
        self._imports: List = []
        self._group = None
        self._token = None
        self._offsets = None
        self._N = 0
        self._plan_stream = None
        self._plan_event = None
        self._owner_planned = False
        self._fwd_planned = None
        self._fwd_plan_event = None
        if world == 1:
            connect_local([self])

    # ------------------------------------------------------------------ wiring
    def _exports(self):
        return (self.weights_dev, self.inbox_ids, self.inbox_counts, self.inbox_grads)

    def _set_peer(self, r: int, ptrs) -> None:
        x = self._x
        x.tables[r], x.inbox_ids[r], x.inbox_counts[r], x.inbox_grads[r] = ptrs

    def connect_processes(self, group: Optional[dist.ProcessGroup] = None) -> None:
        """One process per GPU: map every rank's table and inbox into this process (CUDA IPC) and keep a token for
        the stream-ordered fences."""
        lib = _lib.load()
        self._group = group
        mine = []
        for t in self._exports():
            handle = (C.c_ubyte * 64)()
            off = C.c_int64(0)
            check(lib.recsdk_peer_export(t.data_ptr(), handle, C.byref(off)), "recsdk_peer_export")
            mine.append((bytes(handle), int(off.value)))
        gathered: List = [None] * self.world
        dist.all_gather_object(gathered, mine, group=group)
        for r, entries in enumerate(gathered):
            if r == self.rank:
                self._set_peer(r, [t.data_ptr() for t in self._exports()])
                continue
            ptrs = []
            opened = {}
            for h, off in entries:
                if h not in opened:  # several buffers may share one allocation: open a handle once
                    out = C.c_void_p()
                    buf = (C.c_ubyte * 64).from_buffer_copy(h)
                    check(lib.recsdk_peer_import(buf, 0, C.byref(out)), "recsdk_peer_import")
                    opened[h] = out.value
                    self._imports.append(out.value)
                ptrs.append(opened[h] + off)
            self._set_peer(r, ptrs)
        self._token = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._side_token = torch.zeros(1, dtype=torch.float32, device=self.device)  # fences issued on the side stream
        self._connected = True

    def fence(self) -> None:
        """Stream-ordered barrier across the ranks (a one-element all-reduce); nothing to do for logical ranks of one
        process, whose work is ordered by the stream."""
        if self._token is not None:
            dist.all_reduce(self._token, group=self._group)

    def close(self) -> None:
        """Unmap the peers' buffers (every rank, after the last kernel that uses them has finished)."""
        lib = _lib.load()
        torch.cuda.synchronize(self.device)
        for base in self._imports:
            check(lib.recsdk_peer_release(base, 0), "recsdk_peer_release")
        self._imports = []

    def set_batch_size(self, batch_size: int) -> None:
        """Samples per step of this rank from now on (the buffers were sized at construction: F * batch_size ids must
        fit ``max_ids``)."""
        if self.F * int(batch_size) > self.max_ids and self.pooling_mode != PoolingMode.NONE:
            raise ValueError("batch does not fit the buffers this object was built with")
        self.B = int(batch_size)
        self._x.B = self.B

    # ------------------------------------------------------------------ the step
    def forward(self, indices: torch.Tensor, offsets: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """indices [N] int64 (row ids inside their tables), offsets [F*B+1] feature-major.  Returns the pooled
        [B, F*dim] rows of this rank's samples (NONE pooling: [N, dim])."""
        if not self._connected:
            raise RuntimeError("connect_processes / connect_local first")
        N = indices.numel()
        if offsets.numel() != self.F * self.B + 1:
            raise RuntimeError(f"offset size = {offsets.numel()} is incorrect for feature count = {self.F}, "
                               f"batch {self.B}")
        mode = int(self.pooling_mode)
        shape = (N, self.dim) if mode == _lib.POOL_NONE else (self.B, self.F * self.dim)
        if out is None:
            out = torch.empty(shape, dtype=torch.float32, device=self.device)
        flags = 0
        if self._fwd_planned is not None:
            if self._fwd_planned[:3] != (indices.data_ptr(), N, offsets.data_ptr()):
                raise RuntimeError("the forward plan made ahead belongs to other indices / offsets")
            torch.cuda.current_stream(self.device).wait_event(self._fwd_plan_event)
            self._use(self._fwd_planned[3])  # the scratch the plan was made in is this step's from here on
            self._fwd_planned = None
            flags = 2  # RECSDK_XCHG_FWD_FETCH_ONLY
        check(_lib.load().recsdk_xchg_forward(C.byref(self._x), indices.data_ptr(), offsets.data_ptr(), N, mode,
                                              out.data_ptr(), flags, _stream()), "recsdk_xchg_forward")
        self._offsets, self._N = offsets, N
        return out

    def _use(self, which: int) -> None:
        self._cur = which
        self._ws = self._wss[which]
        self._x.workspace = self._ws.data_ptr()

    def plan_forward_ahead(self, indices: torch.Tensor, offsets: torch.Tensor) -> None:
        """The sort-dedup of the NEXT batch's ids on the side stream, ordered after what is enqueued on the current
        stream so far.  It touches no table and no inbox, so it runs beside whatever the current step still has to do;
        the next forward(indices, offsets) -- exactly these tensors -- then only waits for it and fetches.  Without
        ``double_buffer`` the plan reuses the current step's scratch: call it after backward_local of the current
        batch.  With it the plan goes to the other scratch and may be made any time after the current forward."""
        if not self._connected:
            raise RuntimeError("connect_processes / connect_local first")
        cur = torch.cuda.current_stream(self.device)
        if self._plan_stream is None:
            self._plan_stream = torch.cuda.Stream(device=self.device, priority=-1)
            self._plan_event = torch.cuda.Event()
        if self._fwd_plan_event is None:
            self._fwd_plan_event = torch.cuda.Event()
        self._plan_stream.wait_stream(cur)
        indices.record_stream(self._plan_stream)
        offsets.record_stream(self._plan_stream)
        mine = self._cur
        target = (mine + 1) % len(self._wss)
        self._use(target)
        try:
            check(_lib.load().recsdk_xchg_forward(C.byref(self._x), indices.data_ptr(), offsets.data_ptr(),
                                                  indices.numel(), int(self.pooling_mode), None, 1,
                                                  self._plan_stream.cuda_stream),
                  "recsdk_xchg_forward")  # RECSDK_XCHG_FWD_PLAN_ONLY
        finally:
            self._use(mine)  # the rest of the current step goes on in its own scratch
        self._fwd_plan_event.record(self._plan_stream)
        self._fwd_planned = (indices.data_ptr(), indices.numel(), offsets.data_ptr(), target)

    def backward_local(self, grad_output: torch.Tensor) -> None:
        check(_lib.load().recsdk_xchg_backward_local(C.byref(self._x), grad_output.data_ptr(), self._offsets.data_ptr(),
                                                     self._N, int(self.pooling_mode), int(self.gradient_clipping),
                                                     self.max_gradient, _stream()), "recsdk_xchg_backward_local")

    def _owner_call(self, flags: int, update_events=None, stream=None) -> None:
        ev0 = update_events[0].cuda_event if update_events else None
        ev1 = update_events[1].cuda_event if update_events else None
        h = self.hp
        check(_lib.load().recsdk_xchg_backward_owner(
            C.byref(self._x), self.weights_dev.data_ptr(),
            self.momentum1_dev.data_ptr() if self.momentum1_dev is not None else None,
            self.momentum2_dev.data_ptr() if self.momentum2_dev is not None else None, _OPT_CODE[self.optimizer],
            h["lr"], h["eps"], h["beta1"], h["beta2"], self.iter, ev0, ev1, flags,
            _stream() if stream is None else stream.cuda_stream), "recsdk_xchg_backward_owner")

    def backward_owner(self, update_events=None) -> None:
        """The whole owner phase on the current stream (after the fence that follows backward_local)."""
        self.iter += 1
        if self._owner_planned:
            torch.cuda.current_stream(self.device).wait_event(self._plan_event)
            self._owner_planned = False
            self._owner_call(2, update_events)  # RECSDK_XCHG_OWNER_APPLY_ONLY
        else:
            self._owner_call(0, update_events)

    def plan_owner_ahead(self, fence: bool = False) -> None:
        """The owner phase's index work (compaction of the id lists, sort, runs, records) on a high-priority side
        stream, where it runs beside backward_local; backward_owner then only waits for it and updates the rows.  It
        reads the ids every rank's forward stored into this rank's inbox, so a fence must lie between those forwards
        and it: either the caller's (``fence()`` on the current stream before this call), or -- ``fence=True``, every
        rank alike -- one issued here ON THE SIDE STREAM, which keeps the wait for the slowest rank's forward off the
        stream that runs backward_local (nothing there depends on it)."""
        cur = torch.cuda.current_stream(self.device)
        if self._plan_stream is None:
            self._plan_stream = torch.cuda.Stream(device=self.device, priority=-1)
            self._plan_event = torch.cuda.Event()
        self._plan_stream.wait_stream(cur)
        if fence and self._token is not None:
            with torch.cuda.stream(self._plan_stream):
                dist.all_reduce(self._side_token, group=self._group)
        self._owner_call(1, stream=self._plan_stream)  # RECSDK_XCHG_OWNER_PLAN_ONLY
        self._plan_event.record(self._plan_stream)
        self._owner_planned = True

    def backward(self, grad_output: torch.Tensor, update_events=None, plan_ahead: bool = False) -> None:
        """All backward steps of this rank with the fences between them (every rank calls it).  ``plan_ahead``: one
        more fence (the ids of all ranks are in the inboxes; on the side stream when there are more than two ranks)
        and the owner phase's index work behind it overlaps the local phase."""
        if plan_ahead:
            if self.world > 2:
                self.plan_owner_ahead(fence=True)
            else:  # two ranks are never far apart: the fence on the step's stream measured a little faster there
                self.fence()
                self.plan_owner_ahead()
        self.backward_local(grad_output)
        self.fence()
        self.backward_owner(update_events)
        self.fence()

    def counters(self):
        """(distinct rows asked for, ids received as owner, distinct rows updated, ids in chunked local runs, distinct
        rows asked of this rank itself, chunk sums of the local phase) of the most recent step; synchronises."""
        out = (C.c_int64 * 6)()
        check(_lib.load().recsdk_xchg_counters(C.byref(self._x), out, _stream()), "recsdk_xchg_counters")
        return tuple(int(v) for v in out)

    def raise_if_error(self) -> None:
        raise_on_status(self._status, "DedupExchange")

    # ------------------------------------------------------------------ views of the local table
    def local_table(self, f: int) -> torch.Tensor:
        """[rows, dim] view of this rank's part of table f: the whole table (table-wise; this rank must own it) or
        the rows rank, rank+W, ... (row-wise: local row j is global row j*W + rank)."""
        if self.partition == "table":
            if self.owner_of[f] != self.rank:
                raise ValueError(f"table {f} lives on rank {self.owner_of[f]}")
            start = self._part_base_host[f] - self._rank_base_host[self.rank]
            n = self.rows[f]
        else:
            start = self._part_base_host[self.rank * self.F + f] - self._rank_base_host[self.rank]
            n = self._local_rows_rf[self.rank][f]
        return self.weights_dev[start * self.dim:(start + n) * self.dim].view(n, self.dim)


def connect_local(ranks: Sequence[DedupExchange]) -> None:
    """Wire logical ranks that live in one process: rank r's buffers are addressed with their own pointers (the
    ranks may sit on one GPU, or on several GPUs with peer access enabled).  The caller runs the phases of a step
    for all ranks in order on one stream -- all forwards, all backward_local, all backward_owner -- which is the
    ordering the fences give separate processes."""
    for a in ranks:
        if len(ranks) != a.world:
            raise ValueError("need every rank of the world")
        for b in ranks:
            a._set_peer(b.rank, [t.data_ptr() for t in b._exports()])
        a._connected = True
