"""Table-batched embedding module with the calling convention of the reference's
``HybridSplitTableBatchedEmbeddingBagsCodegen``
(hybrid_torchrec/hybrid_torchrec/distributed/batched_embedding_kernel.py:74-345).

The reference class inherits all of its state from fbgemm_gpu's
``SplitTableBatchedEmbeddingBagsCodegen`` (a third-party package); this module provides the attributes the
reference reads itself (batched_embedding_kernel.py:159-219): ``weights_dev``, ``weights_offsets``,
``D_offsets``, ``total_D``, ``max_D``, ``hash_size_cumsum``, ``total_hash_size_bits``, ``pooling_mode``,
``optimizer``, ``optimizer_args``, ``momentum{1,2}_dev`` (SoA flat tensors), ``iter``, ``dims``, ``step``,
and the swap helpers ``gather_embs`` / ``gather_momentum`` / ``scatter_update_embs`` /
``scatter_update_momentum``.

``forward`` returns an autograd-tracked tensor; its backward runs the fused dedup + segment-sum + sparse
optimizer kernel and updates weights and optimizer state in place (the op returns no weight gradient, like the
reference).  When the torch custom-op library is loaded the call goes through
``torch.ops.fbgemm.split_embedding_codegen_lookup_{adagrad,adam,sgd}_function`` (same schema as the
reference's registration); otherwise through an equivalent ``torch.autograd.Function`` over the same C ABI.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple, Union

import torch
from torch import Tensor, nn

from . import ops

MAX_NUM_EMBEDDINGS = 1_000_000_000  # hybrid_torchrec/constants.py:8-10
MAX_EMBEDDINGS_DIM = 4096


class PoolingMode(enum.IntEnum):
    SUM = 0
    MEAN = 1
    NONE = 2


class EmbOptimType(enum.Enum):
    EXACT_ADAGRAD = "exact_adagrad"
    ADAM = "adam"
    EXACT_SGD = "exact_sgd"


class EmbeddingLocation(enum.IntEnum):
    DEVICE = 0
    MANAGED = 1
    MANAGED_CACHING = 2
    HOST = 3


class ComputeDevice(enum.IntEnum):
    CPU = 0
    CUDA = 1


class SparseType(enum.IntEnum):
    FP32 = 0


_OPT_CODE = {EmbOptimType.EXACT_ADAGRAD: ops.OPT_ADAGRAD, EmbOptimType.ADAM: ops.OPT_ADAM,
             EmbOptimType.EXACT_SGD: ops.OPT_SGD}


@dataclass
class OptimizerArgs:
    stochastic_rounding: bool
    gradient_clipping: bool
    max_gradient: float
    learning_rate: float
    eps: float
    beta1: float
    beta2: float
    weight_decay: float


class _LookupFunction(torch.autograd.Function):
    """Python twin of SplitLookup{Adagrad,Adam,Sgd} (torch_plugin/.../backward_codegen_adam_unweighted_exact.cpp:65-284)."""

    @staticmethod
    def forward(ctx, placeholder, module, indices, offsets, hash_indices, unique_ids, unique_offsets, unique_inverse,
                iteration):
        ctx.module = module
        ctx.iteration = iteration
        ctx.save_for_backward(indices, offsets, hash_indices if hash_indices is not None else torch.empty(0),
                              unique_ids if unique_ids is not None else torch.empty(0),
                              unique_offsets if unique_offsets is not None else torch.empty(0),
                              unique_inverse if unique_inverse is not None else torch.empty(0))
        use = hash_indices if hash_indices is not None else indices
        if module.plan_ahead:  # the backward's index work overlaps this forward on a side stream
            module.plan_backward_ahead(use, offsets, unique_ids, unique_offsets, unique_inverse)
        return module._forward_impl(use, offsets)

    @staticmethod
    def backward(ctx, grad_output):
        indices, offsets, hash_indices, unique_ids, unique_offsets, unique_inverse = ctx.saved_tensors
        m = ctx.module
        use = hash_indices if hash_indices.numel() > 0 else indices
        m._backward_impl(grad_output.contiguous(), use, offsets,
                         unique_ids if unique_ids.numel() > 0 else None,
                         unique_offsets if unique_offsets.numel() > 0 else None,
                         unique_inverse if unique_inverse.numel() > 0 else None, ctx.iteration)
        return (None,) * 9


class HybridSplitTableBatchedEmbeddingBagsCodegen(nn.Module):
    def __init__(
        self,
        embedding_specs: Sequence[Union[Tuple[int, int], Tuple[int, int, EmbeddingLocation, ComputeDevice]]],
        feature_table_map: Optional[List[int]] = None,
        optimizer: EmbOptimType = EmbOptimType.EXACT_SGD,
        pooling_mode: PoolingMode = PoolingMode.SUM,
        weights_precision: SparseType = SparseType.FP32,
        output_dtype: SparseType = SparseType.FP32,
        device: Optional[Union[str, torch.device]] = None,
        learning_rate: float = 0.01,
        eps: float = 1.0e-8,
        beta1: float = 0.9,
        beta2: float = 0.999,
        weight_decay: float = 0.0,
        gradient_clipping: bool = False,
        max_gradient: float = 1.0,
        stochastic_rounding: bool = False,
        initial_accumulator_value: float = 0.0,
        weights_init: Optional[Tuple[float, float]] = None,
        seed: int = 0,
        reduce_chunk: int = 64,
        bounds_check: bool = False,
        use_torch_ops: Optional[bool] = None,
        plan_ahead: bool = False,
        **_ignored,
    ) -> None:
        super().__init__()
        # plan_ahead: every forward also enqueues, on a side stream, the index work of the backward that will
        # follow it (sort of the row keys, runs, per-row records); the backward then only sums and updates.
        # Only for the forward -> backward alternation of training: a second forward before the backward
        # overwrites the plan of the first.
        self.plan_ahead = bool(plan_ahead)
        self._plan_stream = None
        self._plan_event = None
        self._planned_for = None
        if weights_precision != SparseType.FP32 or output_dtype != SparseType.FP32:
            raise ValueError("only fp32 weights/output are supported")
        if not isinstance(optimizer, EmbOptimType):
            raise ValueError(f"Invalid OptimType: {optimizer}")
        self.current_device = torch.device(device if device is not None else "cuda")
        if self.current_device.type != "cuda":
            raise RuntimeError("recsdk_b200 has no CPU path: device must be a CUDA device")
        rows = [int(s[0]) for s in embedding_specs]
        dims = [int(s[1]) for s in embedding_specs]
        for r, d in zip(rows, dims):
            if not (0 < r <= MAX_NUM_EMBEDDINGS) or not (0 < d <= MAX_EMBEDDINGS_DIM):
                raise ValueError(f"invalid table spec ({r}, {d})")
        self.embedding_specs = list(embedding_specs)
        self.rows, self.table_dims = rows, dims
        self.feature_table_map = list(range(len(rows))) if feature_table_map is None else list(feature_table_map)
        T = len(self.feature_table_map)
        self.dims = [dims[t] for t in self.feature_table_map]
        dev = self.current_device

        table_wo = [0]
        table_hs = [0]
        for r, d in zip(rows, dims):
            table_wo.append(table_wo[-1] + r * d)
            table_hs.append(table_hs[-1] + r)
        self.weights_offsets = torch.tensor([table_wo[t] for t in self.feature_table_map], dtype=torch.int64, device=dev)
        d_off = [0]
        for d in self.dims:
            d_off.append(d_off[-1] + d)
        self.D_offsets = torch.tensor(d_off, dtype=torch.int32, device=dev)
        self.total_D, self.max_D = d_off[-1], max(self.dims)
        # per feature, features of one table share the entry; total rows last (fbgemm convention)
        self.hash_size_cumsum = torch.tensor([table_hs[t] for t in self.feature_table_map] + [table_hs[-1]],
                                             dtype=torch.int64, device=dev)
        self.total_hash_size_bits = max(1, int(table_hs[-1]).bit_length())
        self.pooling_mode = PoolingMode(pooling_mode)
        self.optimizer = optimizer
        self.optimizer_args = OptimizerArgs(stochastic_rounding, gradient_clipping, max_gradient, learning_rate, eps,
                                            beta1, beta2, weight_decay)
        self.output_dtype = int(output_dtype)
        self.reduce_chunk = reduce_chunk
        self.bounds_check = bounds_check
        # forward() goes through torch.ops.fbgemm.* (C++ registration) when that library is built; the
        # registered ops use reduce_chunk 64 and no bounds checking, so other settings keep the Python Function
        from . import torch_ops

        if use_torch_ops is None:
            # the registered operators (C++ autograd function, workspace / side stream / events kept per table set)
            # are the default route whenever the library is built; they use reduce_chunk 64 and no bounds checking
            use_torch_ops = torch_ops.available() and reduce_chunk == 64 and not bounds_check
        if use_torch_ops:
            torch_ops.load()
            if plan_ahead:
                # process-wide switch of the registered lookup operators: they plan their own backward ahead
                torch.ops.recsdk.set_plan_ahead(True)
        self.use_torch_ops = bool(use_torch_ops)

        total = table_wo[-1]
        self.weights_dev = nn.Parameter(torch.empty(total, dtype=torch.float32, device=dev), requires_grad=False)
        if weights_init is not None:
            gen = torch.Generator(device=dev)
            gen.manual_seed(seed)
            self.weights_dev.data.uniform_(weights_init[0], weights_init[1], generator=gen)
        else:
            self.weights_dev.data.zero_()
        empty_f = torch.empty(0, dtype=torch.float32, device=dev)
        empty_i = torch.empty(0, dtype=torch.int32, device=dev)
        self.weights_host = torch.empty(0, dtype=torch.float32)
        self.weights_uvm = empty_f
        self.lxu_cache_weights = torch.zeros(0, 0, dtype=torch.float32, device=dev)
        self.weights_placements = torch.zeros(T, dtype=torch.int32, device=dev)
        self.lxu_cache_locations = empty_i
        self.placeholder_autograd_tensor = nn.Parameter(torch.zeros(0, dtype=torch.float32, device=dev))
        n_state = {EmbOptimType.ADAM: 2, EmbOptimType.EXACT_ADAGRAD: 1, EmbOptimType.EXACT_SGD: 0}[optimizer]
        self._optim_num = n_state
        self.momentum1_dev = (torch.full((total,), float(initial_accumulator_value), dtype=torch.float32, device=dev)
                              if n_state >= 1 else empty_f)
        self.momentum2_dev = torch.zeros(total, dtype=torch.float32, device=dev) if n_state >= 2 else empty_f
        for name in ("momentum1", "momentum2"):
            setattr(self, f"{name}_host", torch.empty(0, dtype=torch.float32))
            setattr(self, f"{name}_uvm", empty_f)
            setattr(self, f"{name}_offsets", self.weights_offsets)
            setattr(self, f"{name}_placements", self.weights_placements)
        self.iter = torch.zeros(1, dtype=torch.int64)
        self.step = 0
        self.is_mixed_dim = any(d != self.dims[0] for d in self.dims)
        self._status = ops.new_status(dev)
        self._ws: Optional[Tensor] = None
        self._ws_counters: Optional[Tensor] = None
        self._op_kwargs = None
        self._op = None

    # ------------------------------------------------------------------ kernels
    def _forward_impl(self, indices: Tensor, offsets: Tensor, out: Optional[Tensor] = None, out_shards=None):
        return ops.tbe_forward(self.weights_dev.data, self.weights_offsets, self.D_offsets, indices, offsets,
                               self.total_D, self.max_D, int(self.pooling_mode),
                               status=self._status if self.bounds_check else None, bounds_check=self.bounds_check,
                               out=out, out_shards=out_shards,
                               leave_room=self.plan_ahead and self._planned_for is not None)

    def _ensure_workspace(self, n_indices: int) -> None:
        need = ops.tbe_backward_workspace_bytes(n_indices, self.max_D)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.current_device)

    def plan_backward_ahead(self, indices, offsets, unique_ids=None, unique_offsets=None, unique_inverse=None,
                            grad_shards=None) -> None:
        """Enqueue the index work of the next backward (for exactly these indices / offsets) on the module's side
        stream, ordered after what is already enqueued on the current stream; the backward waits for it."""
        self._ensure_workspace(indices.numel())
        cur = torch.cuda.current_stream(self.current_device)
        if self._plan_stream is None:
            # high priority: the plan's many small kernels take SM slots as the forward's blocks retire instead of
            # queueing behind them
            self._plan_stream = torch.cuda.Stream(device=self.current_device, priority=-1)
            self._plan_event = torch.cuda.Event()
        self._plan_stream.wait_stream(cur)
        for t in (indices, offsets, unique_ids, unique_offsets, unique_inverse):
            if t is not None:
                t.record_stream(self._plan_stream)  # the plan reads them on the side stream
        with torch.cuda.stream(self._plan_stream):
            self._backward_impl(None, indices, offsets, unique_ids, unique_offsets, unique_inverse, 1,
                                grad_shards=grad_shards, phase="plan")
            self._plan_event.record(self._plan_stream)
        self._planned_for = (indices.data_ptr(), indices.numel(), offsets.data_ptr())

    def _backward_impl(self, grad_output, indices, offsets, unique_ids, unique_offsets, unique_inverse, iteration,
                       update_events=None, grad_shards=None, phase: str = "all") -> None:
        a = self.optimizer_args
        self._last_N = indices.numel()  # indices of the most recent backward (bandwidth accounting)
        self._ensure_workspace(indices.numel())
        if phase == "all" and self._planned_for is not None:
            if self._planned_for != (indices.data_ptr(), indices.numel(), offsets.data_ptr()):
                raise RuntimeError("the backward plan made ahead belongs to other indices / offsets")
            torch.cuda.current_stream(self.current_device).wait_event(self._plan_event)
            self._planned_for = None
            phase = "apply"
        ops.tbe_backward(grad_output, self.weights_dev.data,
                         self.momentum1_dev if self._optim_num >= 1 else None,
                         self.momentum2_dev if self._optim_num >= 2 else None,
                         self.weights_offsets, self.D_offsets, self.hash_size_cumsum, indices, offsets, self.total_D,
                         self.max_D, int(self.pooling_mode), _OPT_CODE[self.optimizer], a.learning_rate, a.eps,
                         a.beta1, a.beta2, iteration, unique_ids, unique_offsets, unique_inverse,
                         total_hash_size_bits=self.total_hash_size_bits, reduce_chunk=self.reduce_chunk,
                         gradient_clipping=a.gradient_clipping, max_gradient=a.max_gradient,
                         status=self._status if self.bounds_check else None, bounds_check=self.bounds_check,
                         workspace=self._ws, update_events=update_events, grad_shards=grad_shards, phase=phase)

    # ------------------------------------------------------------------ reference interface
    def forward(self, indices: Tensor, offsets: Tensor, hash_indices: Optional[Tensor] = None,
                unique_indices: Optional[Tensor] = None, unique_offset: Optional[Tensor] = None,
                unique_inverse: Optional[Tensor] = None, per_sample_weights: Optional[Tensor] = None,
                feature_requires_grad: Optional[Tensor] = None,
                batch_size_per_feature_per_rank: Optional[List[List[int]]] = None) -> Tensor:
        if per_sample_weights is not None:
            raise NotImplementedError("weighted lookups are not supported (as in the reference)")
        if batch_size_per_feature_per_rank is not None:
            raise NotImplementedError("variable batch size per feature is not supported")
        indices, offsets = indices.long(), offsets.long()  # prepare_inputs: force_cast_input_types
        self.step += 1
        self.iter[0] += 1  # create_momentum(), batched_embedding_kernel.py:159-176
        iteration = int(self.iter.item())
        if not torch.is_grad_enabled():
            # evaluation / no_grad: no backward will follow, so no lookup function and no plan made ahead
            return self._forward_impl(hash_indices if hash_indices is not None else indices, offsets)
        if self.use_torch_ops:
            return self._invoke_registered_op(indices, offsets, hash_indices, unique_indices, unique_offset,
                                              unique_inverse, iteration)
        return _LookupFunction.apply(self.placeholder_autograd_tensor, self, indices, offsets, hash_indices,
                                     unique_indices, unique_offset, unique_inverse, iteration)

    def _invoke_registered_op(self, indices, offsets, hash_indices, unique_indices, unique_offset, unique_inverse,
                              iteration: int) -> Tensor:
        """The call the reference's invokers make (hybrid_lookup_invoke/hybrid_lookup_{adagrad,adam,sgd}.py):
        torch.ops.fbgemm.split_embedding_codegen_lookup_*_function with the same keyword names."""
        a = self.optimizer_args
        kw = self._op_kwargs
        if kw is None:
            # everything that does not change from call to call, built once
            kw = dict(
                placeholder_autograd_tensor=self.placeholder_autograd_tensor, dev_weights=self.weights_dev.data,
                uvm_weights=self.weights_uvm, lxu_cache_weights=self.lxu_cache_weights,
                weights_placements=self.weights_placements, weights_offsets=self.weights_offsets,
                D_offsets=self.D_offsets, total_D=self.total_D, max_D=self.max_D,
                hash_size_cumsum=self.hash_size_cumsum, total_hash_size_bits=self.total_hash_size_bits,
                pooling_mode=int(self.pooling_mode), indice_weights=None, feature_requires_grad=None,
                lxu_cache_locations=self.lxu_cache_locations, gradient_clipping=a.gradient_clipping,
                max_gradient=a.max_gradient, stochastic_rounding=a.stochastic_rounding, output_dtype=self.output_dtype)
            if self.optimizer != EmbOptimType.EXACT_SGD:
                kw.update(momentum1_dev=self.momentum1_dev, momentum1_uvm=self.momentum1_uvm,
                          momentum1_offsets=self.momentum1_offsets, momentum1_placements=self.momentum1_placements,
                          eps=a.eps)
            if self.optimizer == EmbOptimType.ADAM:
                kw.update(momentum2_dev=self.momentum2_dev, momentum2_uvm=self.momentum2_uvm,
                          momentum2_offsets=self.momentum2_offsets, momentum2_placements=self.momentum2_placements,
                          beta1=a.beta1, beta2=a.beta2, weight_decay=a.weight_decay)
            ns = torch.ops.fbgemm
            self._op = {EmbOptimType.EXACT_ADAGRAD: ns.split_embedding_codegen_lookup_adagrad_function,
                        EmbOptimType.ADAM: ns.split_embedding_codegen_lookup_adam_function,
                        EmbOptimType.EXACT_SGD: ns.split_embedding_codegen_lookup_sgd_function}[self.optimizer]
            self._op_kwargs = kw
        return self._op(indices=indices, offsets=offsets, hash_indices=hash_indices, unique_ids=unique_indices,
                        unique_offsets=unique_offset, unique_inverse=unique_inverse, learning_rate=a.learning_rate,
                        iter=iteration, **kw)

    # swap helpers (batched_embedding_kernel.py:297-345); rows move by bulk copies
    def _check_same_dim(self):
        if self.is_mixed_dim:
            raise ValueError("Mixed dimensions are not supported.")

    def scatter_update_embs(self, indices: Tensor, updates: Tensor) -> None:
        self._check_same_dim()
        ops.scatter_rows(self.weights_dev.data, indices, self.dims[0], updates.reshape(-1))

    def gather_embs(self, indices: Tensor) -> Tensor:
        self._check_same_dim()
        return ops.gather_rows(self.weights_dev.data, indices, self.dims[0]).reshape(-1)

    def gather_momentum(self, indices: Tensor) -> List[Tensor]:
        self._check_same_dim()
        res = []
        if self._optim_num > 0:
            res.append(ops.gather_rows(self.momentum1_dev, indices, self.dims[0]).reshape(-1))
        if self._optim_num > 1:
            res.append(ops.gather_rows(self.momentum2_dev, indices, self.dims[0]).reshape(-1))
        return res

    def scatter_update_momentum(self, indices: Tensor, updates: List[Tensor]) -> None:
        self._check_same_dim()
        if self._optim_num > 0:
            ops.scatter_rows(self.momentum1_dev, indices, self.dims[0], updates[0].reshape(-1))
        if self._optim_num > 1:
            ops.scatter_rows(self.momentum2_dev, indices, self.dims[0], updates[1].reshape(-1))

    def get_momentum(self) -> List[Tensor]:
        res = []
        if self._optim_num > 0:
            res.append(self.momentum1_dev)
        if self._optim_num > 1:
            res.append(self.momentum2_dev)
        return res

    def split_embedding_weights(self) -> List[Tensor]:
        out = []
        off = 0
        for r, d in zip(self.rows, self.table_dims):
            out.append(self.weights_dev.data[off:off + r * d].view(r, d))
            off += r * d
        return out

    def raise_if_error(self) -> None:
        ops.raise_on_status(self._status, "HybridSplitTableBatchedEmbeddingBagsCodegen")

    # ------------------------------------------------------------------ allocation-free stepping (benchmarks, pipelines)
    def forward_into(self, indices: Tensor, offsets: Tensor, out: Optional[Tensor] = None, out_shards=None,
                     plan_grad_shards=None):
        """Forward without autograd bookkeeping, writing into a caller-owned output, or (``out_shards``, an
        ops.SampleShards) straight into the sample owners' peer-mapped buffers.  With ``plan_ahead`` the index work
        of the following backward_from is enqueued on the side stream first (``plan_grad_shards``: the layout that
        backward's gradient will have when it is sample-sharded)."""
        if self.plan_ahead:
            self.plan_backward_ahead(indices, offsets, grad_shards=plan_grad_shards)
        return self._forward_impl(indices, offsets, out=out, out_shards=out_shards)

    def backward_from(self, grad_output: Optional[Tensor], indices: Tensor, offsets: Tensor, unique_indices=None,
                      unique_offset=None, unique_inverse=None, update_events=None, grad_shards=None) -> None:
        """Fused backward + optimizer for the batch of the preceding forward_into.  With ``grad_shards`` the
        gradient rows are read from the sample owners' peer-mapped buffers and ``grad_output`` is None."""
        self.iter[0] += 1
        self._backward_impl(grad_output, indices, offsets, unique_indices, unique_offset, unique_inverse,
                            int(self.iter.item()), update_events=update_events, grad_shards=grad_shards)

    def capture_step(self, indices: Tensor, offsets: Tensor, out: Tensor, grad_output: Tensor) -> "torch.cuda.CUDAGraph":
        """forward_into + backward_from on exactly these tensors as ONE CUDA graph: a step of a small table is a dozen
        short kernels whose launches cost more than their work, and a replay launches them at once.  The caller
        refills ``indices`` / ``offsets`` / ``grad_output`` in place and calls ``.replay()``; ``out`` holds the pooled
        rows after it.  Nothing is executed by the capture.

        Only for optimizers whose scalars do not depend on the step number (Adagrad, SGD): a graph keeps the values
        it was captured with, and Adam's bias correction changes every step.  Call it after at least one ordinary
        step with tensors of these sizes (workspace and side stream exist by then, so the capture allocates nothing),
        with no backward plan pending."""
        if self.optimizer == EmbOptimType.ADAM:
            raise RuntimeError("capture_step: Adam's step-dependent scalars cannot be frozen into a graph")
        if self._ws is None or self._planned_for is not None:
            raise RuntimeError("capture_step: run one ordinary forward_into / backward_from step with these sizes first")
        self._ensure_workspace(indices.numel())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.forward_into(indices, offsets, out)
            self.backward_from(grad_output, indices, offsets)
        return graph

    def last_plan_counters(self) -> Tuple[int, int, int]:
        """(unique rows, chunk sums, indices that live in chunked runs) of the most recent backward (synchronises)."""
        if self._ws is None:
            return 0, 0, 0
        c = self._ws[:64].view(torch.int64)[:3].tolist()
        return int(c[0]), int(c[1]), int(c[2])

    def last_num_unique(self) -> int:
        """Unique rows updated by the most recent backward (synchronises)."""
        return self.last_plan_counters()[0]
