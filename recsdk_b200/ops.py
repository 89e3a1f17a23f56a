"""Functional front end of the C ABI for torch CUDA tensors.

torch is used only for device memory and streams: every function here checks
its arguments, allocates outputs / workspace with torch, and calls one C-ABI
entry point of ``librecsdk_b200.so`` on the current CUDA stream.  There is no
CPU or pure-PyTorch path: CPU tensors are rejected.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import (OPT_ADAGRAD, OPT_ADAM, OPT_SGD, POOL_MEAN, POOL_NONE, POOL_SUM, RecsdkError, check)  # noqa: F401

_STATUS_MESSAGES = {
    _lib.ERR_NEGATIVE_KEY: "Invalid key value: {d0}",
    _lib.ERR_TABLE_FULL: "Ids map reached maxIndex = {d0} please reallocate a larger buffer.",
    _lib.ERR_CACHE_TOO_SMALL: "cacheSize_ too small",
    _lib.ERR_INDEX_RANGE: "row index {d0} out of range (offset {d1})",
    _lib.ERR_HASH_FULL: "key table has no free entry (key {d0})",
    _lib.ERR_TOO_LARGE: "size {d0} beyond the maximum {d1}",
}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    return t.data_ptr()


def _chk(t: torch.Tensor, dtype, name: str) -> torch.Tensor:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (recsdk_b200 has no CPU path)")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} tensor type mismatch: expected {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    return t


def new_status(device) -> torch.Tensor:
    return torch.zeros(_lib.STATUS_WORDS, dtype=torch.int64, device=device)


def raise_on_status(status: torch.Tensor, where: str = "") -> None:
    """Synchronises and raises RuntimeError with the reference's wording when a kernel recorded an error."""
    code, d0, d1, _ = status.tolist()
    if code != 0:
        status.zero_()
        msg = _STATUS_MESSAGES.get(code, _lib.error_string(code)).format(d0=d0, d1=d1)
        err = RecsdkError(code, where)
        err.args = (f"{where}: {msg}" if where else msg,)
        raise err


def _workspace(nbytes: int, device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


# --------------------------------------------------------------------------- A6 forward
class SampleShards:
    """A [B, total_D] matrix stored split by sample over several buffers (one per GPU of the box): sample
    s*shard_B + b is row b of buffer s, rows are ``row_stride`` floats wide and feature t's columns start at
    ``col_offsets[t]`` (int32 device tensor).  ``ptrs`` are device addresses valid on THIS GPU (the local buffer's
    data_ptr and peer mappings of the others, see recsdk_b200.peer)."""

    def __init__(self, ptrs, shard_B: int, row_stride: int, col_offsets: torch.Tensor):
        if not 1 <= len(ptrs) <= _lib.MAX_SHARDS:
            raise RuntimeError(f"1..{_lib.MAX_SHARDS} shards supported, got {len(ptrs)}")
        _chk(col_offsets, torch.int32, "col_offsets")
        self.ptrs, self.shard_B, self.row_stride, self.col_offsets = list(ptrs), shard_B, row_stride, col_offsets

    def fill(self, c_struct) -> None:
        c_struct.num_shards = len(self.ptrs)
        c_struct.row_stride = self.row_stride
        c_struct.shard_B = self.shard_B
        c_struct.col_offsets = _ptr(self.col_offsets)
        for i, q in enumerate(self.ptrs):
            c_struct.ptrs[i] = q


def tbe_forward(dev_weights, weights_offsets, D_offsets, indices, offsets, total_D: int, max_D: int,
                pooling_mode: int, status: Optional[torch.Tensor] = None, bounds_check: bool = True,
                out: Optional[torch.Tensor] = None, out_shards: Optional[SampleShards] = None,
                leave_room: bool = False):
    """With ``out_shards`` the pooled rows are stored into the sample owners' buffers and None is returned."""
    lib = _lib.load()
    _chk(dev_weights, torch.float32, "dev_weights")
    _chk(weights_offsets, torch.int64, "weights_offsets")
    _chk(D_offsets, torch.int32, "D_offsets")
    _chk(indices, torch.int64, "indices")
    _chk(offsets, torch.int64, "offsets")
    T = weights_offsets.numel()
    if T == 0 or (offsets.numel() - 1) % T != 0:
        raise RuntimeError(f"offset size = {offsets.numel()} is incorrect for feature count = {T}")
    B = (offsets.numel() - 1) // T
    N = indices.numel()
    shape = (N, max_D) if pooling_mode == POOL_NONE else (B, total_D)
    if out_shards is not None:
        a = _lib.TbeForwardArgs(_ptr(dev_weights), _ptr(weights_offsets), _ptr(D_offsets), _ptr(indices),
                                _ptr(offsets), None, T, B, N, total_D, max_D, pooling_mode,
                                dev_weights.numel() if bounds_check else 0, _ptr(status))
        out_shards.fill(a.out_shards)
        a.flags = 1 if leave_room else 0  # RECSDK_FWD_LEAVE_ROOM
        check(lib.recsdk_tbe_forward(C.byref(a), _stream()), "recsdk_tbe_forward")
        return None
    if out is None:
        out = torch.empty(shape, dtype=torch.float32, device=dev_weights.device)
    else:
        _chk(out, torch.float32, "out")
        assert tuple(out.shape) == shape
    a = _lib.TbeForwardArgs(_ptr(dev_weights), _ptr(weights_offsets), _ptr(D_offsets), _ptr(indices), _ptr(offsets),
                            _ptr(out), T, B, N, total_D, max_D, pooling_mode,
                            dev_weights.numel() if bounds_check else 0, _ptr(status))
    a.flags = 1 if leave_room else 0  # RECSDK_FWD_LEAVE_ROOM
    check(lib.recsdk_tbe_forward(C.byref(a), _stream()), "recsdk_tbe_forward")
    return out


# --------------------------------------------------------------------------- A1 sorted unique
def unique_sorted(ids: torch.Tensor, key_bits: int = 64,
                  fill: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (unique_buffer[n], inverse[n], num_unique[1]); the first num_unique entries of the buffer are valid.
    ``fill``: value the rest of the buffer is set to beforehand (e.g. INT64_MAX keeps the whole buffer sorted, so it
    can be searched without reading num_unique back)."""
    lib = _lib.load()
    _chk(ids, torch.int64, "ids")
    n = ids.numel()
    dev = ids.device
    uniq = (torch.empty(max(n, 1), dtype=torch.int64, device=dev) if fill is None
            else torch.full((max(n, 1),), fill, dtype=torch.int64, device=dev))
    inv = torch.empty(max(n, 1), dtype=torch.int64, device=dev)
    cnt = torch.zeros(1, dtype=torch.int64, device=dev)
    wsz = lib.recsdk_unique_sorted_workspace_bytes(n)
    ws = _workspace(wsz, dev)
    check(lib.recsdk_unique_sorted(_ptr(ids), n, key_bits, _ptr(uniq), _ptr(inv), _ptr(cnt), _ptr(ws), ws.numel(),
                                   _stream()), "recsdk_unique_sorted")
    return uniq, inv[:n], cnt


def unique_sorted_static(ids: torch.Tensor, unique_out: torch.Tensor, inverse_out: torch.Tensor,
                         num_unique_out: torch.Tensor, key_bits: int = 64) -> None:
    """Sorted unique + inverse into caller-provided outputs with NO device allocation: the sort scratch is
    built into the library (at most ``recsdk_unique_sorted_static_max_n()`` ids).  For callers that must not
    allocate (allocator callbacks, pre-budgeted services).  Calls on one device share that scratch: keep them
    on one stream (or otherwise serialised); make the first call on a device before any stream capture."""
    lib = _lib.load()
    _chk(ids, torch.int64, "ids")
    _chk(unique_out, torch.int64, "unique_out")
    _chk(inverse_out, torch.int64, "inverse_out")
    _chk(num_unique_out, torch.int64, "num_unique_out")
    n = ids.numel()
    if unique_out.numel() < n or inverse_out.numel() < n or num_unique_out.numel() < 1:
        raise RuntimeError("unique_out / inverse_out need n entries and num_unique_out one")
    check(lib.recsdk_unique_sorted_static(_ptr(ids), n, key_bits, _ptr(unique_out), _ptr(inverse_out),
                                          _ptr(num_unique_out), _stream()), "recsdk_unique_sorted_static")


# --------------------------------------------------------------------------- A7 backward
def tbe_backward_workspace_bytes(N: int, max_D: int) -> int:
    return _lib.load().recsdk_tbe_backward_workspace_bytes(N, max_D)


def tbe_backward(grad_output, dev_weights, momentum1, momentum2, weights_offsets, D_offsets, hash_size_cumsum,
                 indices, offsets, total_D: int, max_D: int, pooling_mode: int, optimizer: int,
                 learning_rate: float, eps: float = 0.0, beta1: float = 0.9, beta2: float = 0.999, iter: int = 1,
                 unique_ids=None, unique_offsets=None, unique_inverse=None, total_hash_size_bits: int = 0,
                 reduce_chunk: int = 64, gradient_clipping: bool = False, max_gradient: float = 0.0,
                 status: Optional[torch.Tensor] = None, bounds_check: bool = True,
                 workspace: Optional[torch.Tensor] = None, update_events=None,
                 grad_shards: Optional[SampleShards] = None, staged_update: bool = False,
                 phase: str = "all") -> None:
    """``update_events``: optional (start, stop) torch.cuda.Event pair (created with enable_timing=True and
    recorded at least once before) that the library records around the row-update kernel.
    ``grad_shards``: read the gradient rows from the sample owners' buffers (``grad_output`` is then None).
    ``phase``: "all", or "plan" (index work only; ``grad_output`` may be None; can run on another stream while the
    forward runs) followed later by "apply" with the same arguments and workspace."""
    lib = _lib.load()
    if phase not in ("all", "plan", "apply"):
        raise ValueError(f"phase must be all / plan / apply, got {phase}")
    if grad_shards is None and not (phase == "plan" and grad_output is None):
        _chk(grad_output, torch.float32, "grad_output")
    _chk(dev_weights, torch.float32, "dev_weights")
    if momentum1 is not None:
        _chk(momentum1, torch.float32, "momentum1")
    if momentum2 is not None:
        _chk(momentum2, torch.float32, "momentum2")
    _chk(weights_offsets, torch.int64, "weights_offsets")
    _chk(D_offsets, torch.int32, "D_offsets")
    _chk(indices, torch.int64, "indices")
    _chk(offsets, torch.int64, "offsets")
    have_unique = unique_ids is not None and unique_ids.numel() > 0
    if have_unique:
        _chk(unique_ids, torch.int64, "unique_ids")
        _chk(unique_offsets, torch.int64, "unique_offsets")
        _chk(unique_inverse, torch.int64, "unique_inverse")
    else:
        _chk(hash_size_cumsum, torch.int64, "hash_size_cumsum")
    T = weights_offsets.numel()
    B = (offsets.numel() - 1) // T
    N = indices.numel()
    wsz = lib.recsdk_tbe_backward_workspace_bytes(N, max_D)
    if phase != "all" and (workspace is None or workspace.numel() < wsz):
        raise RuntimeError("plan / apply calls need the caller's workspace (it carries the plan between them)")
    if workspace is None or workspace.numel() < wsz:
        workspace = _workspace(wsz, dev_weights.device)
    a = _lib.TbeBackwardArgs()
    # RECSDK_BWD_STAGED_UPDATE | RECSDK_BWD_PLAN_ONLY | RECSDK_BWD_APPLY_ONLY
    a.flags = (1 if staged_update else 0) | {"all": 0, "plan": 2, "apply": 4}[phase]
    a.grad_output = _ptr(grad_output) if grad_shards is None else None
    if grad_shards is not None:
        grad_shards.fill(a.grad_shards)
    a.dev_weights = _ptr(dev_weights)
    a.momentum1 = _ptr(momentum1)
    a.momentum2 = _ptr(momentum2)
    a.weights_offsets = _ptr(weights_offsets)
    a.D_offsets = _ptr(D_offsets)
    a.hash_size_cumsum = _ptr(hash_size_cumsum) if hash_size_cumsum is not None else None
    a.indices = _ptr(indices)
    a.offsets = _ptr(offsets)
    a.unique_ids = _ptr(unique_ids) if have_unique else None
    a.unique_offsets = _ptr(unique_offsets) if have_unique else None
    a.unique_inverse = _ptr(unique_inverse) if have_unique else None
    a.T, a.B, a.N = T, B, N
    a.num_unique_capacity = unique_ids.numel() if have_unique else 0
    a.total_D, a.max_D = total_D, max_D
    a.pooling_mode, a.optimizer = pooling_mode, optimizer
    a.total_hash_size_bits = total_hash_size_bits
    a.reduce_chunk = reduce_chunk
    a.learning_rate, a.eps, a.beta1, a.beta2 = learning_rate, eps, beta1, beta2
    a.iter = iter
    a.gradient_clipping = int(gradient_clipping)
    a.max_gradient = max_gradient
    a.weights_numel = dev_weights.numel() if bounds_check else 0
    a.dev_status = _ptr(status)
    a.workspace = _ptr(workspace)
    a.workspace_bytes = workspace.numel()
    if update_events is not None:
        a.ev_update_start = update_events[0].cuda_event
        a.ev_update_stop = update_events[1].cuda_event
    check(lib.recsdk_tbe_backward(C.byref(a), _stream()), "recsdk_tbe_backward")


def adam_beta2sqrt(beta1: float, beta2: float, it: int) -> float:
    return _lib.load().recsdk_adam_beta2sqrt(beta1, beta2, it)


# --------------------------------------------------------------------------- A8 rows by slot
def gather_rows(table: torch.Tensor, slots: torch.Tensor, D: int, status=None) -> torch.Tensor:
    lib = _lib.load()
    _chk(table, torch.float32, "table")
    _chk(slots, torch.int64, "slots")
    out = torch.empty((slots.numel(), D), dtype=torch.float32, device=table.device)
    check(lib.recsdk_gather_rows(_ptr(table), _ptr(slots), slots.numel(), D, _ptr(out), table.numel() // D,
                                 _ptr(status), _stream()), "recsdk_gather_rows")
    return out


def scatter_rows(table: torch.Tensor, slots: torch.Tensor, D: int, rows: torch.Tensor, status=None) -> None:
    lib = _lib.load()
    _chk(table, torch.float32, "table")
    _chk(slots, torch.int64, "slots")
    _chk(rows, torch.float32, "rows")
    assert rows.numel() == slots.numel() * D
    check(lib.recsdk_scatter_rows(_ptr(table), _ptr(slots), slots.numel(), D, _ptr(rows), table.numel() // D,
                                  _ptr(status), _stream()), "recsdk_scatter_rows")


# --------------------------------------------------------------------------- A9 TF-flavour ops
def embedding_lookup_by_address(address: torch.Tensor, embedding_dim: int, embedding_type: int = 0) -> torch.Tensor:
    lib = _lib.load()
    _chk(address, torch.int64, "address")
    if embedding_type != 0:
        raise RuntimeError("only fp32 (embedding_type 0) is supported")
    out = torch.empty((address.numel(), embedding_dim), dtype=torch.float32, device=address.device)
    check(lib.recsdk_lookup_by_address(_ptr(address), address.numel(), embedding_dim, _ptr(out), _stream()),
          "recsdk_lookup_by_address")
    return out


def embedding_update_by_address(address: torch.Tensor, embedding: torch.Tensor, update_type: int = 0) -> None:
    lib = _lib.load()
    _chk(address, torch.int64, "address")
    _chk(embedding, torch.float32, "embedding")
    dim = embedding.shape[-1]
    check(lib.recsdk_update_by_address(_ptr(address), address.numel(), dim, _ptr(embedding), update_type,
                                       _stream()), "recsdk_update_by_address")


def lazy_adam(gradient, indices, m, v, var, lr: float, beta1: float, beta2: float, epsilon: float) -> None:
    lib = _lib.load()
    _chk(gradient, torch.float32, "gradient")
    _chk(indices, torch.int32, "indices")
    for t, nme in ((m, "inputM"), (v, "inputV"), (var, "inputVar")):
        _chk(t, torch.float32, nme)
    dim = gradient.shape[-1]
    check(lib.recsdk_lazy_adam(_ptr(gradient), _ptr(indices), indices.numel(), dim, _ptr(m), _ptr(v), _ptr(var), lr,
                               beta1, beta2, epsilon, _stream()), "recsdk_lazy_adam")


def sgd(gradient, indices, var, lr: float, weight_decay: Optional[float] = None) -> None:
    lib = _lib.load()
    _chk(gradient, torch.float32, "gradient")
    _chk(indices, torch.int64, "indices")
    _chk(var, torch.float32, "inputVar")
    dim = gradient.shape[-1]
    ws = _workspace(gradient.numel() * 4, var.device) if weight_decay is not None else None
    check(lib.recsdk_sgd(_ptr(gradient), _ptr(indices), indices.numel(), dim, _ptr(var), lr, weight_decay or 0.0,
                         int(weight_decay is not None), _ptr(ws), ws.numel() if ws is not None else 0, _stream()),
          "recsdk_sgd")


# --------------------------------------------------------------------------- A10 restore
def restore(unique_indices, unique_inverse, unique_offset, offsets_per_table, hash_indices=None) -> torch.Tensor:
    lib = _lib.load()
    _chk(unique_indices, torch.int64, "uniqueIndices")
    _chk(unique_inverse, torch.int64, "uniqueInverse")
    _chk(unique_offset, torch.int64, "uniqueOffset")
    if not isinstance(offsets_per_table, torch.Tensor):
        offsets_per_table = torch.tensor(list(offsets_per_table), dtype=torch.int64, device=unique_inverse.device)
    _chk(offsets_per_table, torch.int64, "offsetsPerTable")
    n = unique_inverse.numel()
    if hash_indices is None:
        hash_indices = torch.empty(n, dtype=torch.int64, device=unique_inverse.device)
    elif hash_indices.numel() != n:
        raise RuntimeError("hashIndices length must equal uniqueInverse length")
    check(lib.recsdk_restore(_ptr(unique_indices), _ptr(unique_inverse), _ptr(unique_offset),
                             _ptr(offsets_per_table), offsets_per_table.numel() - 1, n, _ptr(hash_indices),
                             _stream()), "recsdk_restore")
    return hash_indices


# --------------------------------------------------------------------------- A3 bucketize
def bucketize(lengths, indices, num_features: int, world: int, do_unique: bool = False, return_count: bool = False):
    """Returns (new_lengths[W*F*B], new_indices_buffer[N], unbucketize_permute[N], ids_counts_buffer[N] or None,
    num_out[1]); with do_unique only the first num_out entries of new_indices / ids_counts are valid."""
    lib = _lib.load()
    _chk(lengths, torch.int64, "lengths")
    _chk(indices, torch.int64, "indices")
    if lengths.numel() == 0:
        raise RuntimeError("Lengths tensor is an empty tensor")
    if indices.numel() == 0:
        raise RuntimeError("Indices tensor is an empty tensor")
    if world <= 0:
        raise RuntimeError("Bucket size must be greater than 0")
    dev = indices.device
    n, L = indices.numel(), lengths.numel()
    new_lengths = torch.empty(L * world, dtype=torch.int64, device=dev)
    new_indices = torch.empty(n, dtype=torch.int64, device=dev)
    perm = torch.empty(n, dtype=torch.int64, device=dev)
    counts = torch.empty(n, dtype=torch.int64, device=dev) if (do_unique and return_count) else None
    num_out = torch.zeros(1, dtype=torch.int64, device=dev)
    ws = _workspace(lib.recsdk_bucketize_workspace_bytes(n, L, world), dev)
    check(lib.recsdk_bucketize(_ptr(lengths), L, _ptr(indices), n, num_features, world, int(do_unique),
                               int(return_count), _ptr(new_lengths), _ptr(new_indices), _ptr(perm), _ptr(counts),
                               _ptr(num_out), _ptr(ws), ws.numel(), _stream()), "recsdk_bucketize")
    return new_lengths, new_indices, perm, counts, num_out


# --------------------------------------------------------------------------- jagged-batch utilities
def asynchronous_complete_cumsum(offset: torch.Tensor) -> torch.Tensor:
    """[n] -> [n + 1]: 0 followed by the running sums (asynchronous_complete_cumsum.cpp:18-25)."""
    lib = _lib.load()
    x = offset.to(torch.int64).contiguous()
    n = x.numel()
    out = torch.empty(n + 1, dtype=torch.int64, device=x.device)
    ws = _workspace(lib.recsdk_complete_cumsum_workspace_bytes(n), x.device)
    check(lib.recsdk_complete_cumsum(_ptr(x), n, _ptr(out), _ptr(ws), ws.numel(), _stream()), "recsdk_complete_cumsum")
    return out.to(offset.dtype)


def permute_2D_sparse_data(permute: torch.Tensor, lengths: torch.Tensor, values: torch.Tensor,
                           weights: Optional[torch.Tensor] = None, permuted_lengths_sum: Optional[int] = None):
    """(permuted_lengths [T', B], permuted_values, permuted_weights or None) -- permute2d_sparse_data.cpp:21-48.
    Without ``permuted_lengths_sum`` the output size is read back from the device (one synchronisation), as the
    reference does."""
    lib = _lib.load()
    if lengths.dim() != 2:
        raise RuntimeError("lengths must be 2-D [T, B]")
    if values.element_size() not in (4, 8):
        raise RuntimeError("values must have 4- or 8-byte elements")
    dev = values.device
    perm = permute.to(torch.int64).contiguous()
    len64 = lengths.to(torch.int64).contiguous()
    vals = values.contiguous()
    T_in, B = len64.shape
    T_out = perm.numel()
    w = None
    if weights is not None:
        _chk(weights, torch.float32, "weights")
        if weights.numel() != vals.numel():
            raise RuntimeError(f"weights and values length mismatch: {weights.numel()} vs {vals.numel()}")
        w = weights
    out_len = torch.empty((T_out, B), dtype=torch.int64, device=dev)
    status = new_status(dev)
    ws = _workspace(lib.recsdk_permute_sparse_workspace_bytes(T_in, T_out), dev)
    if permuted_lengths_sum is not None and permuted_lengths_sum > 0:
        total = int(permuted_lengths_sum)
    else:
        total = int(len64.index_select(0, perm).sum().item()) if T_out and B else 0
    out_vals = torch.empty(total, dtype=vals.dtype, device=dev)
    out_w = torch.empty(total, dtype=torch.float32, device=dev) if w is not None else None
    check(lib.recsdk_permute_2d_sparse_data(_ptr(perm), T_out, _ptr(len64), T_in, B, _ptr(vals), vals.element_size(),
                                            _ptr(w), _ptr(out_len), _ptr(out_vals), _ptr(out_w), total, None,
                                            _ptr(status), _ptr(ws), ws.numel(), _stream()),
          "recsdk_permute_2d_sparse_data")
    raise_on_status(status, "permute_2D_sparse_data")
    return out_len.to(lengths.dtype), out_vals, out_w


def permute_1D_sparse_data(permute: torch.Tensor, lengths: torch.Tensor, values: torch.Tensor,
                           weights: Optional[torch.Tensor] = None, permuted_lengths_sum: Optional[int] = None):
    """permute1d_sparse_data.cpp:57-93: the 2-D call on lengths viewed as [L, 1]."""
    if permute.dim() != 1 or lengths.dim() != 1 or values.dim() != 1:
        raise RuntimeError("permute, lengths and values must be 1-D")
    if permuted_lengths_sum is not None and permuted_lengths_sum < 0:
        raise RuntimeError(f"permuted_lengths_sum must be non-negative, got {permuted_lengths_sum}")
    out_len, out_vals, out_w = permute_2D_sparse_data(permute, lengths.view(-1, 1), values, weights, permuted_lengths_sum)
    return out_len.view(-1), out_vals, out_w


def jagged_to_padded_dense(values: torch.Tensor, offsets, max_lengths, padding_value: float = 0.0) -> torch.Tensor:
    """values [N, D], offsets = [tensor [B + 1]] -> [B, max_length, D] (jagged_to_padded_dense.cpp v1 / v2)."""
    lib = _lib.load()
    if not isinstance(offsets, (list, tuple)) or len(offsets) != 1:
        raise RuntimeError(f"offsets must contain exactly 1 tensor, but got {len(offsets)} tensors")
    if isinstance(max_lengths, (list, tuple)):
        if len(max_lengths) != 1:
            raise RuntimeError(f"max_lengths must contain exactly one element, but got {len(max_lengths)}")
        max_lengths = max_lengths[0]
    if max_lengths <= 0:
        raise RuntimeError(f"max_lengths must be positive, but got {max_lengths}")
    _chk(values, torch.float32, "values")
    if values.dim() != 2:
        raise RuntimeError("values must be 2-D")
    offs = offsets[0].to(torch.int64).contiguous()
    B, D = offs.numel() - 1, values.shape[1]
    out = torch.empty((B, int(max_lengths), D), dtype=torch.float32, device=values.device)
    check(lib.recsdk_jagged_to_padded_dense(_ptr(values), _ptr(offs), B, D, int(max_lengths), float(padding_value),
                                            _ptr(out), _stream()), "recsdk_jagged_to_padded_dense")
    return out


def dense_to_jagged(dense: torch.Tensor, offsets, total_L: Optional[int] = None):
    """dense [B, L, D], offsets = [tensor [B + 1]] -> (values [total_L, D], offsets) (dense_to_jagged.cpp); also the
    backward of jagged_to_padded_dense."""
    lib = _lib.load()
    if not isinstance(offsets, (list, tuple)) or len(offsets) != 1:
        raise RuntimeError(f"offsets must contain exactly 1 tensor, but got {len(offsets)} tensors")
    _chk(dense, torch.float32, "dense")
    offs = offsets[0].to(torch.int64).contiguous()
    B, L, D = dense.shape
    if total_L is None:
        total_L = int(offs[-1].item())
    values = torch.empty((total_L, D), dtype=torch.float32, device=dense.device)
    check(lib.recsdk_dense_to_jagged(_ptr(dense), _ptr(offs), B, D, L, _ptr(values), _stream()), "recsdk_dense_to_jagged")
    return values, offsets
