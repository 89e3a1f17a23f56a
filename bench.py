#!/usr/bin/env python
"""Benchmark of the sparse-embedding hot path: one step = pooled gather forward + fused backward
(dedup, gradient segment-sum, sparse Adam) over one synthetic batch of the DLRM-style config
(26 tables, rows log-uniform in [1e3, 4e7] from seed 2025, dim 128 fp32, batch 65536, one id per
field ~ Zipf(1.1), Adam lr 1e-3 beta .9/.999 eps 1e-8).

    python bench.py --gpus N --steps K --warmup W            our arm (CUDA kernels through the C ABI)
    python bench.py --impl reference --gpus N ...            CPU arm: the reference path's CPU restatement
                                                             on the host cores (bounded sample)

Prints ONE JSON line.  `value` = embedding ids/s with inputs resident in HBM; `e2e` = the same metric through
the module API with host index buffers (H2D of indices/offsets and a D2H read of the result inside the timed
region); `roofline` = the row-update kernel's algorithmic bytes / its CUDA-event time against the measured copy
peak; `cpu_baseline` = the CPU oracle on a bounded sample of the same workload.

Multi-GPU (torchrun, one rank per GPU): tables are sharded table-wise by greedy byte balance; every rank runs
the hot path on its own tables for the full batch; pooled outputs go back to the sample owners with one NCCL
all-to-all and the gradients return the same way (weak scaling: per-GPU batch is fixed, the global batch grows).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SEED = 2025
N_TABLES = 26
DIM = 128
BATCH = 65536
ALPHA = 1.1
LR, BETA1, BETA2, EPS = 1e-3, 0.9, 0.999, 1e-8
# Adam state is 3 x rows x 512 B.  The 26 seeded tables hold 144.9 M rows = 222 GB, more than one
# GPU's HBM, so single-GPU runs cap every table at this many rows (Zipf ids are drawn over the capped vocab).
ROW_CAP_1GPU = 16_000_000
UPDATE_KERNEL_DRAM_BYTES = 880_223_488 + 442_036_224
HBM_BUDGET_BYTES = 150e9


def seeded_rows():
    """The 26 row counts of configs[1]: log-uniform in [1e3, 4e7] from the seed (the same draw as
    recsdk_b200.synthetic.table_rows_log_uniform, restated here so that the CPU arm imports nothing of the package)."""
    import numpy as np

    rng = np.random.default_rng(SEED)
    return [int(r) for r in np.round(10 ** rng.uniform(math.log10(1e3), math.log10(4e7), N_TABLES)).astype(np.int64)]


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ============================================================================ our arm
def run_ours(args):
    import torch
    import torch.distributed as dist

    from recsdk_b200 import ops
    from recsdk_b200.synthetic import make_layout, one_hot_batch
    from recsdk_b200.tbe import EmbOptimType, HybridSplitTableBatchedEmbeddingBagsCodegen, PoolingMode

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    rows_all = seeded_rows()
    row_cap = None
    if world == 1:
        row_cap = ROW_CAP_1GPU
        if args.profile_tables > 0:
            # reduced case for profiler captures: the largest tables only, rows capped, so that a few GB are
            # held on the device; the kernels and the batch per table are those of the full workload
            rows_all = sorted(rows_all, reverse=True)[:args.profile_tables]
            row_cap = args.profile_row_cap
        rows_all = [min(r, row_cap) for r in rows_all]
    elif args.profile_tables > 0:
        raise SystemExit("--profile-tables is a 1-GPU option")
    from recsdk_b200.sharding import TableWiseSharding

    sh = TableWiseSharding(rows_all, [DIM] * len(rows_all), world, rank)
    my_tables = sh.local_tables
    rows = [rows_all[t] for t in my_tables]
    state_bytes = sum(rows) * DIM * 4 * 3
    assert state_bytes < HBM_BUDGET_BYTES + 20e9, f"rank {rank}: {state_bytes / 1e9:.1f} GB of table state"
    T = len(rows)
    B = BATCH * world  # a table owner sees the samples of every rank (weak scaling: BATCH per GPU)

    opt_kw = dict(optimizer=EmbOptimType.ADAM, pooling_mode=PoolingMode.SUM, learning_rate=LR, eps=EPS, beta1=BETA1,
                  beta2=BETA2, device=dev, weights_init=(-0.01, 0.01), seed=SEED + rank,
                  plan_ahead=not args.no_plan_ahead)
    module = HybridSplitTableBatchedEmbeddingBagsCodegen([(r, DIM) for r in rows], **opt_kw)
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + 17 * rank)
    n_batches = 4  # rotate distinct batches so consecutive steps touch different rows
    ids_per_step_rank = T * B
    out = torch.empty((B, T * DIM), device=dev, dtype=torch.float32)
    if world == 1:
        batches = [one_hot_batch(gen, rows, B, ALPHA, dev) for _ in range(n_batches)]
        grad = torch.randn((B, T * DIM), generator=gen, device=dev, dtype=torch.float32)
    else:
        # every rank holds the ids of ITS 65536 samples for all 26 fields and the upstream gradient of its
        # samples; ids travel to the table owners, pooled rows come back, gradients go out again
        from recsdk_b200.synthetic import zipf_ids

        # the input pipeline lays the fields out grouped by table owner, so the ids are sent as they lie
        batches = [torch.stack([zipf_ids(gen, BATCH, rows_all[t], ALPHA, dev) for t in sh.output_table_order])
                   .view(N_TABLES, BATCH, 1) for _ in range(n_batches)]
        owner_offsets = torch.arange(T * B + 1, dtype=torch.int64, device=dev)
        if args.exchange == "fused":
            # pooled rows and gradients of this rank's samples live in peer-mapped buffers: the owners' forward
            # kernels store into them and their backward kernels read from them over NVLink
            from recsdk_b200.peer import FusedTableWiseExchange

            del out
            fx = FusedTableWiseExchange(sh, BATCH, dev)
            fx.grads.local.normal_(generator=gen)
            grad = None
        else:
            # upstream gradient of this rank's samples, stored blocked by table owner (what the exchange sends)
            grad = sh.blocked_gradient_buffer(BATCH, dev).normal_(generator=gen)

    ev_pairs = []

    def owner_view(i, ids_local=None):
        """(indices, offsets, upstream gradient) as the table owner sees them for step i."""
        if world == 1:
            idx, offs = batches[i % n_batches]
            return idx, offs, grad
        ids = sh.exchange_ids(batches[i % n_batches] if ids_local is None else ids_local, owner_ordered=True)
        return ids.view(-1), owner_offsets, None

    fused = world > 1 and args.exchange == "fused"
    phase_marks = []  # per timed step: events at the phase boundaries (this rank's stream)
    last_out = [None]

    def step_resident(i, timed=False, idx_offs=None):
        marks = []

        def mark():
            if timed:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                marks.append(e)

        mark()
        idx, offs, g = owner_view(i) if idx_offs is None else (*idx_offs, grad)
        mark()
        evs = None
        if timed:
            evs = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            for e in evs:
                e.record()  # torch creates the CUDA event on first record; the library re-records it
            ev_pairs.append(evs)
            phase_marks.append(marks)
        if fused:
            module.forward_into(idx, offs, out_shards=fx.out_shards, plan_grad_shards=fx.grad_shards)
            mark()
            fx.fence()  # every owner's stores have landed: fx.pooled.local is complete; the dense part runs here
            fx.fence()  # ... and has written fx.grads.local on every rank
            mark()
            module.backward_from(None, idx, offs, update_events=evs, grad_shards=fx.grad_shards)
            mark()
            return
        module.forward_into(idx, offs, out)
        mark()
        if world > 1:
            pooled = sh.exchange_outputs(out, BATCH, assemble=False)  # per-owner [BATCH, D_owner] blocks on the sample owner
            g = sh.exchange_gradients(grad, blocked=True)
            del pooled
        mark()
        module.backward_from(g, idx, offs, update_events=evs)
        mark()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for i in range(args.warmup):
        step_resident(i)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    torch.cuda.cudart().cudaProfilerStart()  # a profiler started with "--profile-from-start off" sees only the timed steps
    t0.record()
    for i in range(args.steps):
        step_resident(args.warmup + i, timed=True)
    t1.record()
    barrier()
    torch.cuda.cudart().cudaProfilerStop()
    ms_total = t0.elapsed_time(t1)
    upd_ms = [a.elapsed_time(b) for a, b in ev_pairs]
    names = ("ids_exchange", "forward", "fences" if fused else "row_exchanges", "backward")
    phases_ms = {n: sum(m[k].elapsed_time(m[k + 1]) for m in phase_marks) / len(phase_marks)
                 for k, n in enumerate(names)}
    U, n_chunks, n_long = module.last_plan_counters()

    # ---- end to end through the module API with host index buffers.  The caller's pipeline double-buffers
    # the H2D copy of the next batch on a copy stream (the reference pipeline's dedicated memcpy stream,
    # torchrec_embcache/distributed/train_pipeline.py:115-119); every step's copy is inside the timed region.
    if world == 1:
        # ids and offsets cross PCIe as int32 (every value fits) and are widened on the device, which is what the
        # reference wrapper's prepare_inputs does with narrower inputs (force_cast_input_types -> .long())
        host = [(idx.to(torch.int32).cpu().pin_memory(), offs.to(torch.int32).cpu().pin_memory()) for idx, offs in batches]
        d_bufs = [(torch.empty_like(batches[0][0], dtype=torch.int32), torch.empty_like(batches[0][1], dtype=torch.int32))
                  for _ in range(2)]
    else:
        host = [(ids.to(torch.int32).cpu().pin_memory(), None) for ids in batches]
        d_bufs = [(torch.empty_like(batches[0], dtype=torch.int32), None) for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    copied = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    result_host = torch.empty(4096, dtype=torch.float32).pin_memory()
    main_stream = torch.cuda.current_stream()
    h2d_bytes = sum(t.numel() * t.element_size() for t in host[0] if t is not None)

    def prefetch(i):
        h_idx, h_offs = host[i % n_batches]
        d_idx, d_offs = d_bufs[i % 2]
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[i % 2])
            d_idx.copy_(h_idx, non_blocking=True)
            if h_offs is not None:
                d_offs.copy_(h_offs, non_blocking=True)
            copied[i % 2].record(copy_stream)

    def step_e2e(i, last):
        if not last:
            prefetch(i + 1)
        d_idx, d_offs = d_bufs[i % 2]
        main_stream.wait_event(copied[i % 2])
        if world == 1:
            if e2e_direct[0]:
                li, lo = d_idx.long(), d_offs.long()
                module.forward_into(li, lo, out)
                module.backward_from(grad, li, lo)
                res = out
            else:
                o = module(d_idx, d_offs)  # autograd-tracked lookup; backward runs the fused optimizer
                o.backward(grad)
                res = o
        elif fused:
            idx, offs, _ = owner_view(i, ids_local=d_idx.long())
            step_resident(i, idx_offs=(idx, offs))
            res = fx.pooled.local
        else:
            idx, offs, _ = owner_view(i, ids_local=d_idx.long())
            o = module(idx, offs)
            res = sh.exchange_outputs(o.detach(), BATCH, assemble=False)[0]
            o.backward(sh.exchange_gradients(grad, blocked=True))
        consumed[i % 2].record(main_stream)
        result_host.copy_(res.detach().reshape(-1)[:4096], non_blocking=True)

    e2e_direct = [False]  # True: the module's stepping API (forward_into / backward_from) instead of autograd

    def run_e2e(n):
        for e in consumed:
            e.record(main_stream)
        prefetch(0)
        for i in range(n):
            step_e2e(i, i == n - 1)

    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e2e_issue_ms = None
    if args.profile_tables > 0:  # profiler captures look at the resident loop only
        e0.record()
        e1.record()
    else:
        # warm-up as long as the timed loop: the host runs ahead of the GPU by up to the whole loop, and the index
        # tensors of the steps in flight (made per step, held back from reuse until the side stream that reads them
        # has passed) must come out of the allocator's pool, not out of cudaMalloc calls inside the timed region
        run_e2e(max(args.warmup, 3, args.steps))
        barrier()
        e0.record()
        t_issue = time.perf_counter()
        run_e2e(args.steps)
        e2e_issue_ms = (time.perf_counter() - t_issue) * 1e3 / args.steps  # host time to enqueue one step
        e1.record()
    barrier()
    e2e_ms_total = e0.elapsed_time(e1)
    e2e_direct_ms = None
    if world == 1 and args.profile_tables == 0:
        # the same loop through the module's stepping API (caller-owned output, no autograd graph)
        e2e_direct[0] = True
        run_e2e(max(args.warmup, 3, args.steps))
        torch.cuda.synchronize()
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d0.record()
        run_e2e(args.steps)
        d1.record()
        torch.cuda.synchronize()
        e2e_direct_ms = d0.elapsed_time(d1) / args.steps
    clocks = sampler.stop() if rank == 0 else None

    # max over ranks
    if world > 1:
        tt = torch.tensor([ms_total, e2e_ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms_total = tt.tolist()
        ids_t = torch.tensor([ids_per_step_rank], device=dev, dtype=torch.float64)
        dist.all_reduce(ids_t)
        ids_per_step = int(ids_t.item())
    else:
        ids_per_step = ids_per_step_rank

    if rank == 0:
        ms_step = ms_total / args.steps
        value = ids_per_step / (ms_step * 1e-3)
        e2e_ms_step = e2e_ms_total / args.steps
        peak, peak_kind = measured_peak_gbs()
        S = 2  # Adam state slots
        N = ids_per_step_rank
        # algorithmic bytes of one row-update launch: per unique row read+write of w, m, v and three 4-byte
        # plan entries; per index that it reduces itself (runs of <= 64) the gradient row and its 4-byte
        # (feature, sample) tag; per chunk sum of a longer run one row of the partial buffer.  The gradient
        # rows of chunked runs are read by partial_kernel and are not counted here.
        upd_bytes = U * (4 * DIM * 2 * (1 + S) + 12) + (N - n_long) * (4 * DIM + 4) + n_chunks * 4 * DIM
        upd_ms_avg = sum(upd_ms) / len(upd_ms)
        achieved = upd_bytes / (upd_ms_avg * 1e-3) / 1e9
        # whole step: dedup (16N + 8U) + forward (N(8+4D) + 8(N+1) + 4D N) + backward (4D N + 8N + 8U + U 4D 2(1+S))
        step_bytes = (16 * N + 8 * U) + (N * (8 + 4 * DIM) + 8 * (N + 1) + 4 * DIM * N) + \
                     (4 * DIM * N + 8 * N + 8 * U + U * 4 * DIM * 2 * (1 + S))
        bits = module.total_hash_size_bits
        passes = min(math.ceil(bits / 8), math.ceil(bits / 9))  # the sort takes 9-bit digits when that saves a pass
        # forward + expand, (scan + scatter) per sort pass, 3 run-scan kernels, records, partial sums, update
        launches_per_step = 1 + (1 + 2 * passes + 3 + 1 + 1 + 1)
        line = {
            "metric": "embedding ids/sec (fwd+bwd+sparse Adam)",
            "value": value,
            "unit": "ids/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f32",
            "data": "synthetic",
            "config": {
                "workload": ("configs[1]: 26 tables dim 128 fp32, batch 65536 per GPU one-hot Zipf(1.1), sparse Adam, "
                             "table-wise sharding") if args.profile_tables == 0 else
                            (f"REDUCED profiling case, not the benchmark: the {T} largest tables of configs[1] with rows "
                             f"capped at {row_cap}, batch 65536, sparse Adam"),
                "tables_this_rank": T, "rows_this_rank": sum(rows), "row_cap": row_cap,
                "table_state_gb_this_rank": round(state_bytes / 1e9, 1),
                "ids_per_step": ids_per_step, "unique_rows_per_step_rank0": U,
                "indices_in_chunked_runs_rank0": n_long, "chunk_sums_rank0": n_chunks,
                "l2": "inputs larger than L2: 872 MB output + 872 MB gradient + 2.6 GB of touched rows per step; "
                      f"{n_batches} distinct batches rotate",
                "reduce_chunk": 64,
                "exchange": ("none (1 GPU)" if world == 1 else
                             "ids: NCCL all-to-all; pooled rows and gradients: peer stores / loads inside the "
                             "forward / backward kernels" if fused else "NCCL all-to-all x3"),
            },
            "step_hbm_gbs": step_bytes / (ms_step * 1e-3) / 1e9,
            "step_hbm_frac_of_measured_peak": step_bytes / (ms_step * 1e-3) / 1e9 / peak,
            "roofline": {"kernel": "update_kernel<Adam>", "bound": "hbm", "achieved": achieved, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                         "bytes_per_launch": upd_bytes, "ms_per_launch": upd_ms_avg,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one update_kernel launch of this workload
                         # (full size, 1 GPU) from a recorded ncu capture; traffic_source says where it comes from
                         "traffic": UPDATE_KERNEL_DRAM_BYTES if (world == 1 and args.profile_tables == 0) else None,
                         "traffic_source": ("ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch, captured on an "
                                            "earlier build of this kernel at the same workload; not re-measured by this run")
                         if (world == 1 and args.profile_tables == 0) else None},
            "e2e": None if args.profile_tables > 0 else
                   {"value": ids_per_step / (e2e_ms_step * 1e-3), "unit": "ids/s", "ms_per_step": e2e_ms_step,
                    "host_enqueue_ms_per_step": e2e_issue_ms, "h2d_bytes_per_step": int(h2d_bytes),
                    "d2h_bytes_per_step": int(result_host.numel() * 4)},
            "e2e_stepping_api": None if e2e_direct_ms is None else
                                {"value": ids_per_step / (e2e_direct_ms * 1e-3), "unit": "ids/s", "ms_per_step": e2e_direct_ms,
                                 "api": "forward_into / backward_from with the same host buffers and copies"},
            "phases_ms_rank0": phases_ms,
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_sample(budget_s=args.cpu_budget)
            line["cpu_baseline_torch"] = cpu_baseline_torch_sample(budget_s=min(8.0, args.cpu_budget))
        emit(line)
    if world > 1:
        dist.barrier()
        if fused:
            fx.close()
            dist.barrier()
        dist.destroy_process_group()




# ============================================================================ N > 1: device-driven dedup exchange
def exchange_parity_check(world, rank, dev):
    """A small seeded twin of the sharded step (same kernels, same process group, same peer mappings) compared bit
    for bit with the CPU oracle of the sharded lookup before anything is timed.  Returns "bit-exact" or a reason."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from oracle import port
    from recsdk_b200.rowwise import TableWiseDedupEmbeddingBag
    from recsdk_b200.tbe import EmbOptimType

    rows, D, B = [3000, 500, 40, 9000, 77], 128, 256
    F = len(rows)
    owner = [f % world for f in range(F)]
    rng = np.random.default_rng(77)
    weights = [rng.uniform(-0.01, 0.01, (r, D)).astype(np.float32) for r in rows]
    batches, grads = [], []
    for q in range(world):
        ids = np.concatenate([np.minimum((rng.pareto(1.1, B) * 3).astype(np.int64), rows[f] - 1) for f in range(F)])
        batches.append((ids.astype(np.int64), np.arange(F * B + 1, dtype=np.int64)))
        grads.append(rng.standard_normal((B, F * D)).astype(np.float32))
    bag = TableWiseDedupEmbeddingBag(rows, D, owner, world, rank, batch_size=B, optimizer=EmbOptimType.ADAM, device=dev,
                                     learning_rate=LR, eps=EPS, beta1=BETA1, beta2=BETA2, one_hot=True)
    orc = port.ShardedDedupOracle(rows, D, world, "table", owner=owner, optimizer=2, lr=LR, eps=EPS, beta1=BETA1,
                                  beta2=BETA2)
    for f, w in enumerate(weights):
        orc.load_table(f, w)
    bag.weights_dev.copy_(torch.from_numpy(orc.w[rank][:bag.weights_dev.numel()]))
    idx, offs = (torch.from_numpy(a).to(dev) for a in batches[rank])
    g = torch.from_numpy(grads[rank]).to(dev)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ok = True
    for _ in range(2):
        exp = orc.step(batches, grads, B, 0)
        out = bag.forward(idx, offs)
        bag.backward(g)
        ok = ok and np.array_equal(out.cpu().numpy(), exp[rank])
    n = bag.weights_dev.numel()
    ok = ok and np.array_equal(bag.weights_dev.cpu().numpy(), orc.w[rank][:n])
    ok = ok and np.array_equal(bag.momentum1_dev.cpu().numpy(), orc.m1[rank][:n])
    ok = ok and np.array_equal(bag.momentum2_dev.cpu().numpy(), orc.m2[rank][:n])
    try:
        bag.raise_if_error()
    except RuntimeError:
        ok = False
    flag = torch.tensor([1.0 if ok else 0.0], device=dev)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        dist.barrier()
        bag.close()
        dist.barrier()
    return "bit-exact" if flag.item() == 1.0 else "MISMATCH against the oracle of the sharded lookup"


def run_dedup_multi(args):
    """configs[1] on N > 1 GPUs: whole tables on ranks, every rank looks up the 26 fields of ITS samples through the
    device-driven dedup exchange (distinct rows pulled from the owners, per-row gradient sums pushed back)."""
    import torch
    import torch.distributed as dist

    from recsdk_b200.rowwise import TableWiseDedupEmbeddingBag
    from recsdk_b200.sharding import greedy_table_placement
    from recsdk_b200.synthetic import zipf_ids
    from recsdk_b200.tbe import EmbOptimType

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    parity = exchange_parity_check(world, rank, dev)

    rows_all = seeded_rows()
    if world == 1:
        # one rank (asked for with --exchange dedup): the exchange kernels with local buffers as "peers"; rows capped
        # as in the default single-GPU run, or to the reduced case for profiler captures
        cap = args.profile_row_cap if args.profile_tables > 0 else ROW_CAP_1GPU
        rows_all = [min(r, cap) for r in rows_all]
    F = len(rows_all)
    if args.placement == "load" and world > 1:
        # what a table costs its owner per step is the distinct rows the ranks ask for, not its share of the ids:
        # count them on one profile batch (same seed on every rank, not one of the timed batches) and balance those
        pg = torch.Generator(device=dev)
        pg.manual_seed(SEED + 4242)
        loads = [int(torch.unique(zipf_ids(pg, BATCH, rows_all[t], ALPHA, dev)).numel()) for t in range(F)]
        owner = greedy_table_placement(rows_all, [DIM] * F, world, loads=loads, bytes_cap=150 * 10**9)
    else:
        owner = greedy_table_placement(rows_all, [DIM] * F, world)
    bag = TableWiseDedupEmbeddingBag(rows_all, DIM, owner, world, rank, batch_size=BATCH, optimizer=EmbOptimType.ADAM,
                                     device=dev, learning_rate=LR, eps=EPS, beta1=BETA1, beta2=BETA2,
                                     weights_init=(-0.01, 0.01), seed=SEED + rank, one_hot=True,
                                     double_buffer=(args.fwd_plan == "early"))
    state_bytes = bag.local_rows * DIM * 4 * 3
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + 17 * rank)
    n_batches = 4
    main_stream = torch.cuda.current_stream()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def allreduce_max(t):
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t

    # where the fence before the owner's plan goes: measured, the side stream wins with 4 and 8 ranks (1.15 vs 1.21 and
    # 1.19 vs 1.32 ms), the step's own stream with 2 (1.06 vs 1.08 ms)
    owner_plan = args.owner_plan
    if owner_plan == "auto":
        owner_plan = "ahead" if world > 2 else "ahead_main_fence"

    def measure(B, profile=False):
        """One scaling mode: B samples per rank.  Returns a dict of timings.  `profile`: a profiler started with
        --profile-from-start off sees the resident loop only (not the generation of the batches)."""
        bag.set_batch_size(B)
        batches = [torch.stack([zipf_ids(gen, B, rows_all[t], ALPHA, dev) for t in range(F)]).view(-1)
                   for _ in range(n_batches)]
        offsets = torch.arange(F * B + 1, dtype=torch.int64, device=dev)
        grad = torch.randn((B, F * DIM), generator=gen, device=dev, dtype=torch.float32)
        out = torch.empty((B, F * DIM), device=dev, dtype=torch.float32)
        ev_pairs, marks_all = [], []

        def step(i, timed=False, ids=None, next_ids=None):
            """One step on `ids` (default: the resident batch i).  `next_ids`: a callable that returns the ids tensor
            of the following step, or None; with --fwd-plan ahead its sort-dedup is enqueued on the side stream as
            soon as this step's local backward phase no longer needs the scratch."""
            marks = []

            def mark():
                if timed:
                    e = torch.cuda.Event(enable_timing=True)
                    e.record()
                    marks.append(e)

            evs = None
            if timed:
                evs = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                for e in evs:
                    e.record()
                ev_pairs.append(evs)
                marks_all.append(marks)
            mark()
            if timed and bag._fwd_planned is not None:
                # what the forward would wait for anyway, timed on its own: the sort-dedup made ahead on the side stream
                main_stream.wait_event(bag._fwd_plan_event)
            mark()
            bag.forward(batches[i % n_batches] if ids is None else ids, offsets, out=out)
            mark()
            if owner_plan == "ahead":
                # a fence (the ids of every rank are in the owners' inboxes) and the owner phase's index work, both on
                # the side stream, beside the local phase
                bag.plan_owner_ahead(fence=True)
            elif owner_plan == "ahead_main_fence":
                bag.fence()  # the same with the fence on the stream of the step
                bag.plan_owner_ahead()
            if args.fwd_plan == "early" and next_ids is not None:
                bag.plan_forward_ahead(next_ids(), offsets)  # second scratch: beside the local phase already
            bag.backward_local(grad)
            if args.fwd_plan == "ahead" and next_ids is not None:
                bag.plan_forward_ahead(next_ids(), offsets)  # beside the fences and the owner phase
            mark()
            bag.fence()
            mark()
            bag.backward_owner(evs)
            mark()
            bag.fence()
            mark()

        total = args.warmup + args.steps

        def resident_next(i):
            return (lambda: batches[(i + 1) % n_batches]) if i + 1 < total else None

        if profile:
            barrier()
            torch.cuda.cudart().cudaProfilerStart()
        for i in range(args.warmup):
            step(i, next_ids=resident_next(i))
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(args.steps):
            step(args.warmup + i, timed=True, next_ids=resident_next(args.warmup + i))
        t1.record()
        barrier()
        if profile:
            torch.cuda.cudart().cudaProfilerStop()
        ms_total = t0.elapsed_time(t1)
        names = ("wait_for_forward_plan", "forward", "backward_local", "fence", "backward_owner", "fence2")
        phases = {n: sum(m[k].elapsed_time(m[k + 1]) for m in marks_all) / len(marks_all) for k, n in enumerate(names)}
        upd_ms = sum(a.elapsed_time(b) for a, b in ev_pairs) / len(ev_pairs)
        counters = bag.counters()
        bag.raise_if_error()
        # what one fence costs when nobody is late: 20 back to back on an idle stream
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(20):
            bag.fence()
        f1.record()
        barrier()
        fence_idle_ms = f0.elapsed_time(f1) / 20
        phases_all = [phases]
        if world > 1:
            phases_all = [None] * world
            dist.all_gather_object(phases_all, phases)

        # end to end: ids of every step cross PCIe from pinned host memory (int32, widened on the device) on a copy
        # stream, double-buffered; 16 KB of the result are read back
        host = [b.to(torch.int32).cpu().pin_memory() for b in batches]
        d_bufs = [torch.empty_like(batches[0], dtype=torch.int32) for _ in range(2)]
        copy_stream = torch.cuda.Stream(device=dev)
        copied = [torch.cuda.Event(), torch.cuda.Event()]
        consumed = [torch.cuda.Event(), torch.cuda.Event()]
        result_host = torch.empty(4096, dtype=torch.float32).pin_memory()

        def prefetch(i):
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[i % 2])
                d_bufs[i % 2].copy_(host[i % n_batches], non_blocking=True)
                copied[i % 2].record(copy_stream)

        def run_e2e(n):
            for e in consumed:
                e.record(main_stream)
            prefetch(0)
            main_stream.wait_event(copied[0])
            cur_ids = d_bufs[0].long()
            consumed[0].record(main_stream)
            for i in range(n):
                if i + 1 < n:
                    prefetch(i + 1)
                nxt = [None]

                def widen_next(j=i + 1):
                    # the next batch's ids are on the device (double-buffered copy): widen them now so that their
                    # sort-dedup can be planned beside this step's owner phase
                    main_stream.wait_event(copied[j % 2])
                    nxt[0] = d_bufs[j % 2].long()
                    consumed[j % 2].record(main_stream)
                    return nxt[0]

                step(i, ids=cur_ids, next_ids=widen_next if i + 1 < n else None)
                if i + 1 < n:
                    cur_ids = nxt[0] if nxt[0] is not None else widen_next()
                result_host.copy_(out.reshape(-1)[:4096], non_blocking=True)

        run_e2e(max(args.warmup, 3, args.steps))  # as long as the timed loop, see the single-GPU loop
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        t_issue = time.perf_counter()
        run_e2e(args.steps)
        issue_ms = (time.perf_counter() - t_issue) * 1e3 / args.steps
        e1.record()
        barrier()
        tt = allreduce_max(torch.tensor([ms_total, e0.elapsed_time(e1)], device=dev, dtype=torch.float64))
        cc = allreduce_max(torch.tensor([counters[0] - counters[4]], device=dev, dtype=torch.float64))  # rows that crossed
        return dict(ms_step=tt[0].item() / args.steps, e2e_ms_step=tt[1].item() / args.steps, phases=phases,
                    phases_all=phases_all, fence_idle_ms=fence_idle_ms,
                    upd_ms=upd_ms, counters=counters, issue_ms=issue_ms, h2d=int(host[0].numel() * 4),
                    remote_rows_max=int(cc.item()), B=B)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    weak = measure(BATCH, profile=True)
    clocks = sampler.stop() if rank == 0 else None
    strong = measure(BATCH // world) if world > 1 else weak  # the config as written: a global batch of 65536 split over the ranks

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        S = 2
        U_req, n_recv, U_own, n_long, U_self, n_chunks = weak["counters"]
        ids_per_step = F * BATCH * world
        # row update on the owner: per distinct row read+write of w, m, v and its 32-byte record; per received id
        # one gradient row of the inbox and its 4-byte slot number
        upd_bytes = U_own * (4 * DIM * 2 * (1 + S) + 32) + n_recv * (4 * DIM + 4)
        achieved = upd_bytes / (weak["upd_ms"] * 1e-3) / 1e9
        # this rank's HBM traffic by the step formula: its own N ids looked up (dedup, rows written to the pooled output,
        # gradients read once), plus the update of the rows it owns
        N = F * BATCH
        step_bytes = (16 * N + 8 * U_req) + (U_req * 4 * DIM + 8 * (N + 1) + 4 * DIM * N) + \
                     (4 * DIM * N + 8 * N + U_req * 4 * DIM) + (n_recv * (8 + 4 * DIM) + U_own * 4 * DIM * 2 * (1 + S))
        # bytes that cross NVLink per step and GPU, each direction: one row per distinct remote row pulled in the
        # forward, one summed gradient row per distinct remote row pushed in the backward (+ 8 bytes of id)
        remote = weak["remote_rows_max"]
        nv_in, nv_out = remote * DIM * 4, remote * (DIM * 4 + 8)
        ph = weak["phases"]
        nv_in_gbs = nv_in / (ph["forward"] * 1e-3) / 1e9
        nv_out_gbs = nv_out / (ph["backward_local"] * 1e-3) / 1e9
        passes = min(math.ceil(bag.key_bits / b) for b in (8, 9, 10))
        passes_o = min(math.ceil(max(1, int(bag.local_rows).bit_length()) / b) for b in (8, 9, 10))
        launches_per_step = (1 + 2 * passes + 3 + 3) + 2 + (1 + 2 * passes_o + 3 + 2)

        def scal(m, label):
            ids = F * m["B"] * world
            return {"scaling": label, "batch_per_gpu": m["B"], "ids_per_step": ids, "ms_per_step": m["ms_step"],
                    "value": ids / (m["ms_step"] * 1e-3), "e2e_value": ids / (m["e2e_ms_step"] * 1e-3),
                    "phases_ms_rank0": m["phases"]}

        line = {
            "metric": "embedding ids/sec (fwd+bwd+sparse Adam)", "value": ids_per_step / (weak["ms_step"] * 1e-3),
            "unit": "ids/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": weak["ms_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {
                "workload": "configs[1]: 26 tables dim 128 fp32, batch 65536 per GPU one-hot Zipf(1.1), sparse Adam, "
                            "table-wise sharding",
                "placement": (args.placement if world > 1 else None), "tables_per_rank": [owner.count(r) for r in range(world)],
                "tables_this_rank": owner.count(rank), "rows_this_rank": bag.local_rows,
                "row_cap": None if world > 1 else max(rows_all),
                "table_state_gb_this_rank": round(state_bytes / 1e9, 1), "ids_per_step": ids_per_step,
                "distinct_rows_requested_rank0": U_req, "ids_received_as_owner_rank0": n_recv,
                "distinct_rows_updated_rank0": U_own,
                "l2": "inputs larger than L2: 872 MB output + 872 MB gradient + touched rows per step; "
                      f"{n_batches} distinct batches rotate",
                "reduce_chunk": 64,
                "exchange": "device-driven dedup exchange over peer mappings: distinct ids and counts stored into the "
                            "owners' inboxes, distinct rows loaded from the owners' tables, per-row gradient sums stored "
                            "into the owners' inboxes, counts read on the device; two one-element NCCL all-reduces per "
                            "step as fences" + (", a third one after the forward, on the side stream, so that the owner phase's "
                                                "index work runs beside the local backward phase" if owner_plan == "ahead" else
                                               (", a third one after the forward so that the owner phase's index work runs "
                                                "beside the local backward phase" if owner_plan == "ahead_main_fence" else "")),
                "owner_plan": owner_plan, "fwd_plan": args.fwd_plan,
            },
            "parity_check": parity,
            "step_hbm_gbs_rank0": step_bytes / (weak["ms_step"] * 1e-3) / 1e9,
            "step_hbm_frac_of_measured_peak": step_bytes / (weak["ms_step"] * 1e-3) / 1e9 / peak,
            "roofline": {"kernel": "update_kernel<Adam> (owner phase)", "bound": "hbm", "achieved": achieved, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak, "bytes_per_launch": upd_bytes,
                         "ms_per_launch": weak["upd_ms"], "traffic": None},
            "nvlink": {"bytes_per_step_per_gpu": {"in": nv_in, "out": nv_out},
                       "gbs": {"in_over_forward_phase": nv_in_gbs, "out_over_backward_local_phase": nv_out_gbs},
                       "frac_of_900": max(nv_in_gbs, nv_out_gbs) / 900.0,
                       "frac_of_measured_770": max(nv_in_gbs, nv_out_gbs) / 770.0,
                       "note": "per direction; the phases also hold the sort / pooling work, so these are lower bounds "
                               "of the link rate while rows move"},
            "e2e": {"value": ids_per_step / (weak["e2e_ms_step"] * 1e-3), "unit": "ids/s",
                    "ms_per_step": weak["e2e_ms_step"], "host_enqueue_ms_per_step": weak["issue_ms"],
                    "h2d_bytes_per_step": weak["h2d"], "d2h_bytes_per_step": 4096 * 4},
            "phases_ms_rank0": weak["phases"],
            "phases_ms_min_max_over_ranks": {k: [min(p[k] for p in weak["phases_all"]), max(p[k] for p in weak["phases_all"])]
                                             for k in weak["phases"]},
            "phases_ms_per_rank": [{k: round(v, 4) for k, v in p.items()} for p in weak["phases_all"]],
            "fence_ms_when_idle": weak["fence_idle_ms"],
            "strong_scaling": scal(strong, "strong: global batch 65536 split over the ranks"),
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        emit(line)
    if world > 1:
        dist.barrier()
        bag.close()
        dist.barrier()
        dist.destroy_process_group()



# ============================================================================ the other configs (--config c1|c3|c4|c5)
def _time_loop(torch, fn, steps, warmup):
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()  # a profiler started with "--profile-from-start off" sees only timed steps
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    t0 = time.perf_counter()
    for i in range(steps):
        fn(warmup + i)
    issue_ms = (time.perf_counter() - t0) * 1e3 / steps
    b.record()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    return a.elapsed_time(b) / steps, issue_ms


def run_tbe_config(args, name):
    """configs[0] (c1: one table 1e6 x 16, batch 4096 one-hot Zipf(1.05), Adagrad acc 0.1) and configs[2] (c3: 26 tables
    of 1e6..1e7 rows x 64, batch 16384, bag length U[1,100], Zipf(1.2), SUM, Adagrad) on one GPU: forward + fused
    backward through the module's stepping calls, end to end with host index buffers, the row-update kernel against
    the measured copy peak, and the CPU restatement beside it."""
    import numpy as np
    import torch

    from recsdk_b200.synthetic import multi_hot_batch, one_hot_batch
    from recsdk_b200.tbe import EmbOptimType, HybridSplitTableBatchedEmbeddingBagsCodegen, PoolingMode

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if name == "c1":
        rows, D, B, alpha, max_len, seed, init = [1_000_000], 16, 4096, 1.05, 1, 1234, 0.05
        label = "configs[0]: one table 1e6 x 16 fp32, batch 4096 one-hot Zipf(1.05), sparse Adagrad lr 0.01 acc 0.1"
    else:
        rng = np.random.default_rng(7)
        rows = [int(r) for r in np.round(10 ** rng.uniform(6, 7, 26)).astype(np.int64)]
        D, B, alpha, max_len, seed, init = 64, 16384, 1.2, 100, 7, 0.05
        label = ("configs[2]: 26 tables of 1e6..1e7 rows (log-uniform, seed 7) x 64 fp32, batch 16384, bag length "
                 "U[1,100], ids Zipf(1.2), SUM pooling, sparse Adagrad lr 0.01 acc 0.1")
    T = len(rows)
    module = HybridSplitTableBatchedEmbeddingBagsCodegen(
        [(r, D) for r in rows], optimizer=EmbOptimType.EXACT_ADAGRAD, pooling_mode=PoolingMode.SUM, device=dev,
        learning_rate=0.01, eps=1e-8, initial_accumulator_value=0.1, weights_init=(-init, init), seed=seed,
        plan_ahead=not args.no_plan_ahead)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    n_batches = 4
    batches = [one_hot_batch(gen, rows, B, alpha, dev) if max_len == 1 else multi_hot_batch(gen, rows, B, max_len, alpha, dev)
               for _ in range(n_batches)]
    grad = torch.randn((B, T * D), generator=gen, device=dev)
    out = torch.empty((B, T * D), device=dev)
    ev_pairs = []

    def step(i, timed=False):
        idx, offs = batches[i % n_batches]
        evs = None
        if timed:
            evs = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            for e in evs:
                e.record()
            ev_pairs.append(evs)
        module.forward_into(idx, offs, out)
        module.backward_from(grad, idx, offs, update_events=evs)

    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    ms_step, _ = _time_loop(torch, lambda i: step(i, timed=True), args.steps, args.warmup)
    upd_ms = sum(a.elapsed_time(b) for a, b in ev_pairs[-args.steps:]) / args.steps
    U, n_chunks, n_long = module.last_plan_counters()
    N = int(np.mean([b[0].numel() for b in batches]))

    # end to end through module(indices, offsets) + backward with pinned host index buffers (int32 on the wire)
    host = [(i.to(torch.int32).cpu().pin_memory(), o.to(torch.int32).cpu().pin_memory()) for i, o in batches]
    result_host = torch.empty(min(4096, B * T * D), dtype=torch.float32).pin_memory()

    def step_e2e(i):
        hi, ho = host[i % n_batches]
        o = module(hi.to(dev, non_blocking=True), ho.to(dev, non_blocking=True))
        o.backward(grad)
        result_host.copy_(o.detach().reshape(-1)[:result_host.numel()], non_blocking=True)

    e2e_ms, issue_ms = _time_loop(torch, step_e2e, args.steps, max(args.warmup, 3, args.steps))  # pool warm, see run_ours
    without_graph = None
    if name == "c1":
        # the step is a dozen kernels of a few microseconds: replayed as ONE CUDA graph (static index / offset buffers
        # refilled every step: device-to-device for `value`, from pinned host memory for `e2e`)
        s_idx, s_offs = batches[0][0].clone(), batches[0][1].clone()
        graph = module.capture_step(s_idx, s_offs, out, grad)

        def step_graph(i):
            idx, offs = batches[i % n_batches]
            s_idx.copy_(idx)
            s_offs.copy_(offs)
            graph.replay()

        def step_graph_e2e(i):
            hi, ho = host[i % n_batches]
            s_idx.copy_(hi, non_blocking=True)
            s_offs.copy_(ho, non_blocking=True)
            graph.replay()
            result_host.copy_(out.reshape(-1)[:result_host.numel()], non_blocking=True)

        without_graph = {"ms_per_step": ms_step, "e2e_ms_per_step": e2e_ms, "host_enqueue_ms_per_step": issue_ms}
        ms_step, _ = _time_loop(torch, step_graph, args.steps, max(args.warmup, 3))
        e2e_ms, issue_ms = _time_loop(torch, step_graph_e2e, args.steps, max(args.warmup, 3))
    clocks = sampler.stop()
    peak, peak_kind = measured_peak_gbs()
    S = 1
    upd_bytes = U * (4 * D * 2 * (1 + S) + 32) + (N - n_long) * (4 * D + 4) + n_chunks * 4 * D
    bags = T * B
    step_bytes = (16 * N + 8 * U) + (N * (8 + 4 * D) + 8 * (bags + 1) + 4 * D * bags) + \
                 (4 * D * bags + 8 * N + 8 * U + U * 4 * D * 2 * (1 + S))
    line = {
        "metric": "embedding ids/sec (fwd+bwd+sparse Adagrad)", "value": N / (ms_step * 1e-3), "unit": "ids/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "us_per_step": ms_step * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": label, "ids_per_step": N, "bags_per_step": bags, "unique_rows_per_step": U,
                   "table_state_gb": round(sum(rows) * D * 4 * 2 / 1e9, 2),
                   "l2": (f"{n_batches} distinct batches rotate; " +
                          ("the step moves ~0.6 MB: launch / latency bound, the roofline fraction is informational"
                           if name == "c1" else "output + gradient + touched rows per step exceed L2"))},
        "step_hbm_gbs": step_bytes / (ms_step * 1e-3) / 1e9,
        "step_hbm_frac_of_measured_peak": step_bytes / (ms_step * 1e-3) / 1e9 / peak,
        "roofline": {"kernel": "update_kernel<Adagrad>", "bound": "hbm", "achieved": upd_bytes / (upd_ms * 1e-3) / 1e9,
                     "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": upd_bytes / (upd_ms * 1e-3) / 1e9 / peak,
                     "bytes_per_launch": upd_bytes, "ms_per_launch": upd_ms, "traffic": None},
        "e2e": {"value": N / (e2e_ms * 1e-3), "unit": "ids/s", "ms_per_step": e2e_ms, "host_enqueue_ms_per_step": issue_ms,
                "h2d_bytes_per_step": int(host[0][0].numel() * 4 + host[0][1].numel() * 4),
                "d2h_bytes_per_step": int(result_host.numel() * 4)},
        "gpu_launches": (1 + 1 + 2 * 3 + 3 + 1 + 1 + 1) * args.steps,
        "clocks": clocks,
    }
    if without_graph is not None:
        line["config"]["step"] = "forward + fused backward captured once as a CUDA graph and replayed (13 kernels per replay)"
        line["without_graph"] = without_graph
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = _cpu_tbe_config(name, rows, D, B, alpha, max_len, args.cpu_budget)
    emit(line)


def _cpu_tbe_config(name, rows, D, B, alpha, max_len, budget_s):
    """The CPU restatement on the same shapes; c3's tables are capped at 262144 rows and the batch at 2048 samples so
    that the sample stays within the time budget (c1 runs at full size)."""
    import numpy as np

    from oracle import port

    cores = os.cpu_count() or 1
    port.set_num_threads(cores)
    rng = np.random.default_rng(3)
    if name != "c1":
        rows, B = [min(r, 262_144) for r in rows], 2048
    T = len(rows)
    wo = np.concatenate([[0], np.cumsum([r * D for r in rows])]).astype(np.int64)
    do = (np.arange(T + 1) * D).astype(np.int32)
    hs = np.concatenate([[0], np.cumsum(rows)]).astype(np.int64)
    w = rng.uniform(-0.05, 0.05, int(wo[-1])).astype(np.float32)
    acc = np.full_like(w, 0.1)
    lens = np.ones(T * B, np.int64) if max_len == 1 else rng.integers(1, max_len + 1, T * B)
    idx = []
    for t, r in enumerate(rows):
        n = int(lens[t * B:(t + 1) * B].sum())
        p = np.arange(1, r + 1, dtype=np.float64) ** (-alpha)
        cdf = np.cumsum(p)
        idx.append(np.minimum(np.searchsorted(cdf, rng.random(n) * cdf[-1]), r - 1))
    idx = np.concatenate(idx).astype(np.int64)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    grad = rng.standard_normal((B, T * D)).astype(np.float32)

    def one():
        port.tbe_forward(w, wo[:-1].copy(), do, idx, offs, T, B, T * D, D, 0)
        port.tbe_backward(grad, w, acc, None, wo[:-1].copy(), do, hs, idx, offs, T, B, T * D, D, 0, 1, 0.01, 1e-8,
                          reduce_chunk=64)

    one()
    t0, n = time.perf_counter(), 0
    while time.perf_counter() - t0 < budget_s and n < 200:
        one()
        n += 1
    dt = time.perf_counter() - t0
    return {"value": idx.size * n / dt, "unit": "ids/s", "cores": cores, "kind": "port",
            "sample": f"{n} steps of {T} table(s) with rows capped at {max(rows)} x {B} samples ({idx.size} ids per step), "
                      "oracle C restatement with OpenMP"}


def run_c4(args):
    """configs[3]: dynamic hash-keyed table, 64 Mi slots x 32 fp32, 131072 keys per step with 30 % new keys, admission
    at count >= 2, eviction of keys idle for more than 50 steps every 10 steps, gather + sparse Adam on the cache rows.
    One step = timestamps -> counts -> first-occurrence unique -> admission filter -> slot policy (-> evict) -> pooled
    gather over the slots -> fused backward.  Before timing, the slots of the first steps are compared with the CPU
    restatement of SwapManager + FeatureFilter (or the reference's compiled classes when oracle/_ref holds them)."""
    import numpy as np
    import torch

    from recsdk_b200 import ops
    from recsdk_b200.embcache import AdmitAndEvictConfig, EmbcacheManager, EmbConfig
    from recsdk_b200.tbe import EmbOptimType, HybridSplitTableBatchedEmbeddingBagsCodegen, PoolingMode

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    cache, D, n_keys, interval, thr = 64 << 20, 32, 131072, 10, 50
    total_steps = args.warmup + 2 * args.steps + 10  # parity steps, warm-up, timed steps, end-to-end steps
    rng = np.random.default_rng(99)
    issued = rng.integers(0, 2**63 - 1, size=n_keys, dtype=np.int64)
    stream = []
    for _ in range(total_steps):
        fresh = rng.integers(0, 2**63 - 1, size=int(n_keys * 0.3), dtype=np.int64)
        keys = np.concatenate([fresh, issued[rng.integers(0, issued.size, size=n_keys - fresh.size)]])
        rng.shuffle(keys)
        issued = np.concatenate([issued, fresh])
        stream.append(keys)
    cfg = EmbConfig("dyn", emb_dim=D, optim_num=2, cache_size=cache, weight_init_max=1.0,
                    admit_and_evict_config=AdmitAndEvictConfig(2, 0.0, thr, interval), filter_capacity=1 << 26)
    mgr = EmbcacheManager([cfg], device=dev)
    module = HybridSplitTableBatchedEmbeddingBagsCodegen([(cache, D)], optimizer=EmbOptimType.ADAM,
                                                        pooling_mode=PoolingMode.SUM, device=dev, learning_rate=LR, eps=EPS,
                                                        beta1=BETA1, beta2=BETA2, weights_init=(-0.01, 0.01), seed=99)
    d_stream = [torch.from_numpy(k).to(dev) for k in stream]
    offsets = torch.arange(n_keys + 1, dtype=torch.int64, device=dev)
    grad = torch.randn((n_keys, D), device=dev)
    out = torch.empty((n_keys, D), device=dev)

    h_stream = None  # pinned host copies of the key batches, made for the end-to-end loop only

    def step(i, from_host=False):
        k = h_stream[i].to(dev, non_blocking=True) if from_host else d_stream[i]
        ts = torch.full_like(k, i)
        offs2 = [0, n_keys]
        mgr.record_timestamp(k, offs2, ts)
        if i > 0 and (i + 1) % interval == 0:
            mgr.evict_features()
            mgr.remove_embedding_table_info()
        mgr.feature_filters[0].StatisticsKeyCount(k)
        uq, inv, cnt = ops.unique_sorted(k)  # the CPU side of the slot check dedups in the same (ascending) order
        n_u = int(cnt.item())
        info = mgr.compute_swap_info(uq[:n_u].contiguous(), [0, n_u])
        slots = info.batch_offs[inv]
        module.forward_into(slots, offsets, out)
        module.backward_from(grad, slots, offsets)
        return uq, info

    # ---- slot parity on the first steps against the CPU classes
    from oracle import port, ref

    try:
        have_ref = ref.available() and ref.embcache() is not None
    except OSError:
        have_ref = False
    cs, cf = (ref.SwapManager(cache, 1), ref.FeatureFilter(2, thr, interval)) if have_ref else \
             (port.SwapManager(cache, 1), port.FeatureFilter(2, thr, interval))
    parity = "bit-exact"
    for i in range(min(8, total_steps)):
        uq, info = step(i)
        k = stream[i]
        cf.record_timestamp(k, np.full(k.size, i, np.int64))
        cf.statistics_key_count(k)
        res = cs.compute_swap_info(cf.count_filter(np.unique(k)))
        exp_offs = np.asarray(res[4] if isinstance(res, (tuple, list)) else res["batch_offs"])
        if not np.array_equal(info.batch_offs.cpu().numpy(), exp_offs):
            parity = f"MISMATCH of slots at step {i}"
            break
    it = [8]

    def timed(_):
        step(it[0])
        it[0] += 1

    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    ms_step, issue_ms = _time_loop(torch, timed, args.steps, args.warmup)
    # end to end: the same steps (the key stream goes on) with every batch of keys crossing PCIe from pinned host memory
    # inside the timed region; the step reads its two counts back anyway
    first_e2e = it[0]
    h_stream = {j: stream[j] for j in range(first_e2e, total_steps)}
    h_stream = {j: torch.from_numpy(a).pin_memory() for j, a in h_stream.items()}
    e2e_steps = max(1, min(args.steps, total_steps - first_e2e - 1))

    def timed_e2e(_):
        step(it[0], from_host=True)
        it[0] += 1

    e2e_ms, e2e_issue_ms = _time_loop(torch, timed_e2e, e2e_steps, 1)
    clocks = sampler.stop()
    peak, peak_kind = measured_peak_gbs()
    U = int(ops.unique_sorted(d_stream[it[0] - 1])[2].item())
    S = 2
    step_bytes = (16 * n_keys + 8 * U) + 16 * n_keys + (n_keys * (8 + 4 * D) + 8 * (n_keys + 1) + 4 * D * n_keys) + \
                 (4 * D * n_keys + 8 * n_keys + 8 * U + U * 4 * D * 2 * (1 + S))
    line = {
        "metric": "embedding ids/sec (key->slot + fwd+bwd+sparse Adam)", "value": n_keys / (ms_step * 1e-3), "unit": "ids/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int64 keys / f32 rows", "data": "synthetic",
        "config": {"workload": "configs[3]: dynamic hash-keyed table, 64 Mi slots x 32 fp32, 131072 keys per step, 30 % "
                               "new keys, admit at count >= 2, evict idle > 50 steps every 10 steps, gather + sparse Adam",
                   "ids_per_step": n_keys, "unique_keys_last_step": U,
                   "host_reads_per_step": "two (unique count, swap counts): the reference's interface returns host lists"},
        "parity_check": parity + (" (slots of the first 8 steps vs the reference's compiled SwapManager + FeatureFilter)"
                                  if have_ref else " (slots of the first 8 steps vs the CPU restatement)"),
        "step_hbm_gbs": step_bytes / (ms_step * 1e-3) / 1e9,
        "roofline": {"kernel": "whole step (policy phases are latency bound)", "bound": "hbm",
                     "achieved": step_bytes / (ms_step * 1e-3) / 1e9, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": step_bytes / (ms_step * 1e-3) / 1e9 / peak, "traffic": None},
        "e2e": {"value": n_keys / (e2e_ms * 1e-3), "unit": "ids/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
                "host_enqueue_ms_per_step": e2e_issue_ms, "h2d_bytes_per_step": n_keys * 8, "d2h_bytes_per_step": 32,
                "note": "keys from pinned host memory every step; the step reads two counts back"},
        "clocks": clocks,
    }
    emit(line)


def run_c5(args):
    """configs[4]: one row-wise sharded table, 1e9 rows x 64 fp32 with Adam state at 8 GPUs (1.25e8 rows per GPU at any
    N: 5e8 at 4, 2.5e8 at 2, 1.25e8 at 1), batch 262144 one-hot ids ~ Zipf(1.05) per GPU, through the device-driven
    dedup exchange with rows placed by id % W."""
    import torch
    import torch.distributed as dist

    from recsdk_b200.rowwise import RowWiseShardedEmbeddingBag
    from recsdk_b200.tbe import EmbOptimType

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rows, D, B, alpha = 125_000_000 * world, 64, 262144, 1.05
    bag = RowWiseShardedEmbeddingBag([rows], D, world, rank, batch_size=B, optimizer=EmbOptimType.ADAM, device=dev,
                                     learning_rate=LR, eps=EPS, beta1=BETA1, beta2=BETA2, weights_init=(-0.01, 0.01),
                                     seed=5 + rank, one_hot=True)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5 + 17 * rank)

    def zipf_large(n):
        # inverse of the continuous Zipf CDF (a 1e9-entry table of exact probabilities would not fit beside the
        # rows): rank = (1 + u (V^(1-a) - 1))^(1/(1-a)); ranks spread over the ids by a multiplicative hash
        u = torch.rand(n, generator=gen, dtype=torch.float64, device=dev)
        r = (1.0 + u * (float(rows) ** (1.0 - alpha) - 1.0)).pow(1.0 / (1.0 - alpha)).to(torch.int64).clamp_(1, rows) - 1
        return (r * 2654435761 + 12345) % rows

    batches = [zipf_large(B) for _ in range(4)]
    offsets = torch.arange(B + 1, dtype=torch.int64, device=dev)
    grad = torch.randn((B, D), generator=gen, device=dev)
    out = torch.empty((B, D), device=dev)

    def step(i):
        bag.forward(batches[i % 4], offsets, out=out)
        bag.backward(grad)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(args.steps):
        step(args.warmup + i)
    t1.record()
    barrier()
    ms = torch.tensor([t0.elapsed_time(t1) / args.steps], device=dev, dtype=torch.float64)
    host = [b.cpu().pin_memory() for b in batches]
    result_host = torch.empty(4096, dtype=torch.float32).pin_memory()

    def step_e2e(i):
        bag.forward(host[i % 4].to(dev, non_blocking=True), offsets, out=out)
        bag.backward(grad)
        result_host.copy_(out.reshape(-1)[:4096], non_blocking=True)

    for i in range(3):
        step_e2e(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step_e2e(i)
    e1.record()
    barrier()
    e2e = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
    counters = bag.counters()
    bag.raise_if_error()
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        ms_step, e2e_ms = ms.item(), e2e.item()
        U_req, n_recv, U_own, _, U_self, _ = counters
        S = 2
        step_bytes = (16 * B + 8 * U_req) + (U_req * 4 * D + 8 * (B + 1) + 4 * D * B) + (4 * D * B + 8 * B + U_req * 4 * D) + \
                     (n_recv * (8 + 4 * D) + U_own * 4 * D * 2 * (1 + S))
        remote = U_req - U_self
        emit({
            "metric": "embedding ids/sec (fwd+bwd+sparse Adam)", "value": B * world / (ms_step * 1e-3), "unit": "ids/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"configs[4]: row-wise sharded table, {rows} rows x 64 fp32 + Adam state over {world} GPU(s) "
                                   "(1.25e8 rows = 96 GB per GPU), batch 262144 one-hot ids ~ Zipf(1.05) per GPU, rows "
                                   "placed by id % W, device-driven dedup exchange",
                       "ids_per_step": B * world, "distinct_rows_requested_rank0": U_req,
                       "distinct_rows_updated_rank0": U_own,
                       "ids": "continuous inverse-CDF Zipf sampler (an exact 1e9-entry CDF does not fit beside the rows)"},
            "step_hbm_gbs_rank0": step_bytes / (ms_step * 1e-3) / 1e9,
            "roofline": {"kernel": "whole step of rank 0 (sort / scan phases are latency bound at this batch size)",
                         "bound": "hbm", "achieved": step_bytes / (ms_step * 1e-3) / 1e9, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": step_bytes / (ms_step * 1e-3) / 1e9 / peak,
                         "traffic": None},
            "nvlink": {"bytes_per_step_per_gpu": {"in": remote * D * 4, "out": remote * (D * 4 + 8)}},
            "e2e": {"value": B * world / (e2e_ms * 1e-3), "unit": "ids/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": 4096 * 4},
            "clocks": clocks,
        })
    if world > 1:
        dist.barrier()
        bag.close()
        dist.barrier()
        dist.destroy_process_group()


# ============================================================================ per-operator measurements
def run_ops(args):
    """`--workload ops`: every other entry point of the path (dedup, key tables, cache policy, bucketize, row
    moves, TF-flavour optimizers, restore) timed on the GPU at the sizes the configs give them, with the CPU
    implementation timed beside it on the same inputs: the reference's own compiled classes where oracle/_ref holds
    them ("reference"), else the C restatement ("port").  Small ops (a few MB) are launch- and latency-bound; the
    bandwidth fraction is printed for orientation only.  One JSON line."""
    import numpy as np
    import torch

    from oracle import port, ref
    from recsdk_b200 import FeatureFilter, IdsMapper, SwapManager, ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peak, peak_kind = measured_peak_gbs()
    rng = np.random.default_rng(SEED)
    res = {}

    def gpu_ms(fn, iters=20, warm=3, setup=None):
        for i in range(warm):
            if setup:
                setup(i)
            fn(i)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if setup is None:
            a.record()
            for i in range(iters):
                fn(warm + i)
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / iters
        tot = 0.0
        for i in range(iters):
            setup(warm + i)
            a.record()
            fn(warm + i)
            b.record()
            torch.cuda.synchronize()
            tot += a.elapsed_time(b)
        return tot / iters

    def cpu_ms(fn, iters=3):
        fn(0)
        t0 = time.perf_counter()
        for i in range(iters):
            fn(1 + i)
        return (time.perf_counter() - t0) / iters * 1e3

    def entry(name, n, unit, g_ms, c_ms, kind, alg_bytes):
        res[name] = {"n": n, "unit": unit, "gpu_ms": g_ms, "gpu_per_s": n / (g_ms * 1e-3), "cpu_ms": c_ms,
                     "cpu_kind": kind, "cpu_per_s": n / (c_ms * 1e-3), "algorithmic_bytes": alg_bytes,
                     "gbs": alg_bytes / (g_ms * 1e-3) / 1e9, "frac_of_peak": alg_bytes / (g_ms * 1e-3) / 1e9 / peak}

    try:
        have_ref = ref.available() and ref.embcache() is not None
    except OSError:
        have_ref = False

    # ---- A1 sorted unique + inverse: the ids of one configs[1] step (26 x 65536, linearised, 28-bit keys)
    rows = [min(r, ROW_CAP_1GPU) for r in seeded_rows()]
    base = np.concatenate([[0], np.cumsum(rows)])[:-1]
    ids_np = np.concatenate([base[t] + np.minimum((rng.pareto(1.1, BATCH) * 10).astype(np.int64), rows[t] - 1)
                             for t in range(N_TABLES)]).astype(np.int64)
    ids = torch.from_numpy(ids_np).to(dev)
    bits = int(sum(rows)).bit_length()
    g = gpu_ms(lambda i: ops.unique_sorted(ids, key_bits=bits))
    u = int(ops.unique_sorted(ids, key_bits=bits)[2].item())
    c = cpu_ms(lambda i: port.unique_sorted(ids_np))
    entry("unique_sorted", ids_np.size, "ids", g, c, "port", 16 * ids_np.size + 8 * u)

    # ---- A2 IdsMapper.ids2indices_unique: dynamic-table config, 131072 keys per step, 30 % new
    n_keys, steps = 131072, 26
    issued = rng.integers(0, 2**62, size=n_keys, dtype=np.int64)
    stream = []
    for s_ in range(steps):
        fresh = rng.integers(0, 2**62, size=int(n_keys * 0.3), dtype=np.int64)
        keys = np.concatenate([fresh, issued[rng.integers(0, issued.size, size=n_keys - fresh.size)]])
        rng.shuffle(keys)
        issued = np.concatenate([issued, fresh])
        stream.append(keys)
    d_stream = [torch.from_numpy(k).to(dev) for k in stream]
    gm = IdsMapper(64 << 20, True, device=dev)
    g = gpu_ms(lambda i: gm.ids2indices_unique(d_stream[i], check=False))
    if have_ref:
        t = ref.load_hybrid()
        cm = t.classes.hybrid.IdsMapper(64 << 20, True)
        c_stream = [torch.from_numpy(k) for k in stream]
        c = cpu_ms(lambda i: cm.ids2indices_unique(c_stream[i]), iters=5)
        kind = "reference"
    else:
        cm = port.IdsMapper(64 << 20, True)
        c = cpu_ms(lambda i: cm.ids2indices_unique(stream[i]), iters=5)
        kind = "port"
    entry("ids_mapper_ids2indices_unique", n_keys, "keys", g, c, kind, n_keys * (8 + 16 + 24))

    # ---- A4 + A5 cache policy step (record_timestamp, statistics, count_filter, compute_swap_info)
    gs, gf = SwapManager(64 << 20, 1, device=dev), FeatureFilter("t", 2, 50, 10, capacity=1 << 24, device=dev)

    def gpu_policy(i):
        k = d_stream[i]
        ts = torch.full_like(k, i)
        gf.RecordTimestamp(k, ts)
        gf.StatisticsKeyCount(k)
        uq_buf, _, uq_n = ops.unique_sorted(k)  # the caller's dedup (sorted here; order does not change the work)
        uq = uq_buf[:int(uq_n.item())]
        gf.CountFilter(uq)
        gs.ComputeSwapInfoDevice(uq)

    g = gpu_ms(gpu_policy)
    if have_ref:
        cs, cf, kind = ref.SwapManager(64 << 20, 1), ref.FeatureFilter(2, 50, 10), "reference"
    else:
        cs, cf, kind = port.SwapManager(64 << 20, 1), port.FeatureFilter(2, 50, 10), "port"

    def cpu_policy(i):
        k = stream[i]
        cf.record_timestamp(k, np.full(k.size, i, np.int64))
        cf.statistics_key_count(k)
        uq = np.unique(k)
        cs.compute_swap_info(cf.count_filter(uq))

    c = cpu_ms(cpu_policy, iters=5)
    entry("cache_policy_step", n_keys, "keys", g, c, kind, n_keys * (32 * 2 + 16 + 40))

    # ---- A3 bucketize: row-wise config, 262144 ids, 8 buckets, with dedup
    nb, Fb, Wb = 262144, 4, 8
    b_idx = rng.integers(0, 10**9, size=nb, dtype=np.int64)
    b_idx[: nb // 2] = b_idx[nb // 2:][: nb // 2] % 100000
    b_len = np.ones(nb, np.int64)
    d_idx, d_len = torch.from_numpy(b_idx).to(dev), torch.from_numpy(b_len).to(dev)
    g = gpu_ms(lambda i: ops.bucketize(d_len, d_idx, Fb, Wb, do_unique=True, return_count=True))
    if have_ref:
        t = ref.load_hybrid()
        ci, cl = torch.from_numpy(b_idx), torch.from_numpy(b_len)
        c = cpu_ms(lambda i: t.ops.hybrid.block_bucketize_sparse_features_cpu(
            cl, ci, False, True, torch.ones(Fb, dtype=torch.int64), Wb, None, None, None, 0, None, False, False, True, True))
        kind = "reference"
    else:
        c = cpu_ms(lambda i: port.bucketize(b_len, b_idx, Fb, Wb, do_unique=True, return_count=True))
        kind = "port"
    entry("bucketize_unique", nb, "ids", g, c, kind, nb * (8 + 8 + 8 + 8))

    # ---- A8 swap rows: gather + scatter of 65536 rows of 128 floats out of a 4 M-row table
    D, k_rows, t_rows = DIM, 65536, 4 << 20
    table = torch.empty(t_rows * D, device=dev).uniform_(-1, 1)
    slots = torch.randperm(t_rows, device=dev)[:k_rows].contiguous()
    buf = ops.gather_rows(table, slots, D)

    def swap_rows(i):
        r = ops.gather_rows(table, slots, D)
        ops.scatter_rows(table, slots, D, r)

    g = gpu_ms(swap_rows)
    t_np, s_np = table[: (1 << 20) * D].cpu().numpy(), (slots % (1 << 20)).cpu().numpy()
    c = cpu_ms(lambda i: port.scatter_rows(t_np, s_np, D, port.gather_rows(t_np, s_np, D)))
    entry("gather_plus_scatter_rows", k_rows, "rows", g, c, "port", k_rows * D * 4 * 4)

    # ---- A9 LazyAdam on 65536 rows of 128
    idx32 = slots.to(torch.int32)
    m_t, v_t = torch.zeros_like(table), torch.zeros_like(table)
    grad = torch.randn(k_rows, D, device=dev)
    g = gpu_ms(lambda i: ops.lazy_adam(grad, idx32, m_t, v_t, table, 1e-3, 0.9, 0.999, 1e-8))
    g_np, i_np = grad.cpu().numpy(), (idx32 % (1 << 20)).cpu().numpy()
    var_np, m_np, v_np = t_np.copy(), np.zeros_like(t_np), np.zeros_like(t_np)
    c = cpu_ms(lambda i: port.lazy_adam(g_np, i_np, m_np, v_np, var_np, 1e-3, 0.9, 0.999, 1e-8))
    entry("lazy_adam", k_rows, "rows", g, c, "port", k_rows * D * 4 * 7)

    # ---- A10 restore: hash_indices[r] = unique[inverse[r] + offset[t]] over one configs[1] step
    uq, inv, cnt = ops.unique_sorted(ids, key_bits=bits)
    uoff = torch.tensor([0, u], dtype=torch.int64, device=dev)
    per_table = torch.tensor([0, ids.numel()], dtype=torch.int64, device=dev)
    g = gpu_ms(lambda i: ops.restore(uq, inv, uoff, per_table))
    uq_np, inv_np = uq.cpu().numpy(), inv.cpu().numpy()
    c = cpu_ms(lambda i: port.restore(uq_np, inv_np, np.array([0, u], np.int64), np.array([0, ids_np.size], np.int64)))
    entry("restore", ids_np.size, "ids", g, c, "port", ids_np.size * 24)

    # ---- jagged-batch utilities on the configs[1] batch shape: 26 x 65536 lengths, 1.7 M values
    kl = np.ones((N_TABLES, BATCH), np.int64)
    kp = rng.permutation(N_TABLES).astype(np.int32)
    d_kl, d_kp = torch.from_numpy(kl).to(dev), torch.from_numpy(kp).to(dev)
    g = gpu_ms(lambda i: ops.permute_2D_sparse_data(d_kp, d_kl, ids, None, ids.numel()))
    c = cpu_ms(lambda i: port.permute_2D_sparse_data(kp, kl, ids_np))
    entry("permute_2D_sparse_data", ids_np.size, "values", g, c, "port", ids_np.size * 8 * 4)
    flat_l = d_kl.view(-1)
    g = gpu_ms(lambda i: ops.asynchronous_complete_cumsum(flat_l))
    c = cpu_ms(lambda i: port.asynchronous_complete_cumsum(kl.reshape(-1)))
    entry("asynchronous_complete_cumsum", kl.size, "lengths", g, c, "port", kl.size * 16)
    jl = rng.integers(0, 101, 16384)
    jo = np.concatenate([[0], np.cumsum(jl)]).astype(np.int64)
    jv = torch.randn(int(jo[-1]), 64, device=dev)
    d_jo = torch.from_numpy(jo).to(dev)
    g = gpu_ms(lambda i: ops.jagged_to_padded_dense(jv, [d_jo], 100, 0.0))
    jv_np = jv.cpu().numpy()
    c = cpu_ms(lambda i: port.jagged_to_padded_dense(jv_np, jo, 100, 0.0))
    entry("jagged_to_padded_dense", int(jo[-1]), "rows", g, c, "port", int(jo[-1]) * 256 + 16384 * 100 * 256)

    emit({"workload": "ops", "n_gpus": 1, "peak_gbs": peak, "peak_kind": peak_kind, "cores": os.cpu_count(),
          "data": "synthetic", "ops": res})

# ============================================================================ CPU arms (oracle)
CPU_SAMPLE_ROW_CAP = 262_144
CPU_SAMPLE_BATCH = 8192


def _cpu_sample_setup():
    """Bounded sample of the workload for the CPU legs: all 26 tables with rows capped at 262144
    (4.4 GB of fp32 Adam state) and 8192 of the 65536 samples per step."""
    import numpy as np

    from oracle import port

    rows = [min(r, CPU_SAMPLE_ROW_CAP) for r in seeded_rows()]
    T, B = len(rows), CPU_SAMPLE_BATCH
    rng = np.random.default_rng(SEED)
    wo = np.concatenate([[0], np.cumsum([r * DIM for r in rows])]).astype(np.int64)
    do = (np.arange(T + 1) * DIM).astype(np.int32)
    hs = np.concatenate([[0], np.cumsum(rows)]).astype(np.int64)
    w = rng.uniform(-0.01, 0.01, int(wo[-1])).astype(np.float32)
    m1 = np.zeros_like(w)
    m2 = np.zeros_like(w)
    idx = []
    for r in rows:
        p = np.arange(1, r + 1, dtype=np.float64) ** (-ALPHA)
        cdf = np.cumsum(p)
        u = rng.random(B) * cdf[-1]
        idx.append(np.minimum(np.searchsorted(cdf, u), r - 1))
    idx = np.concatenate(idx).astype(np.int64)
    offs = np.arange(T * B + 1, dtype=np.int64)
    grad = rng.standard_normal((B, T * DIM)).astype(np.float32)
    return port, dict(T=T, B=B, wo=wo[:-1].copy(), do=do, hs=hs, w=w, m1=m1, m2=m2, idx=idx, offs=offs, grad=grad)


def _cpu_step(port, c, it):
    out = port.tbe_forward(c["w"], c["wo"], c["do"], c["idx"], c["offs"], c["T"], c["B"], c["T"] * DIM, DIM, 0)
    port.tbe_backward(c["grad"], c["w"], c["m1"], c["m2"], c["wo"], c["do"], c["hs"], c["idx"], c["offs"], c["T"],
                      c["B"], c["T"] * DIM, DIM, 0, 2, LR, EPS, BETA1, BETA2, it)
    return out


def cpu_baseline_sample(budget_s: float = 15.0):
    port, c = _cpu_sample_setup()
    cores = os.cpu_count() or 1
    port.set_num_threads(cores)  # explicit: a launcher's OMP_NUM_THREADS=1 must not decide the baseline
    _cpu_step(port, c, 1)
    t0 = time.perf_counter()
    n = 0
    while time.perf_counter() - t0 < budget_s and n < 50:
        _cpu_step(port, c, n + 2)
        n += 1
    dt = time.perf_counter() - t0
    ids = c["T"] * c["B"] * n
    return {"value": ids / dt, "unit": "ids/s", "cores": cores, "kind": "port",
            "sample": f"{n} steps of 26 tables (rows capped at {CPU_SAMPLE_ROW_CAP}) x {CPU_SAMPLE_BATCH} samples, "
                      "oracle C restatement with OpenMP (forward + fused backward + Adam)"}


def cpu_baseline_torch_sample(budget_s: float = 8.0):
    """The stock PyTorch CPU path on the same bounded sample: one nn.EmbeddingBag(mode="sum", sparse=True) per table and
    torch.optim.SparseAdam -- what the reference's own operator tests use as their golden
    (cust_op/.../test_split_embedding_codegen_lookup_function.py:149-170).  Reported beside the C restatement, not
    instead of it.  (SparseAdam's update differs from the fused kernel's in the last bits; this leg is a timing.)"""
    import numpy as np
    import torch

    rows = [min(r, CPU_SAMPLE_ROW_CAP) for r in seeded_rows()]
    T, B = len(rows), CPU_SAMPLE_BATCH
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    rng = np.random.default_rng(SEED)
    bags = [torch.nn.EmbeddingBag(r, DIM, mode="sum", sparse=True) for r in rows]
    for b in bags:
        torch.nn.init.uniform_(b.weight, -0.01, 0.01)
    opt = torch.optim.SparseAdam([b.weight for b in bags], lr=LR, betas=(BETA1, BETA2), eps=EPS)
    idx = []
    for r in rows:
        p = np.arange(1, r + 1, dtype=np.float64) ** (-ALPHA)
        cdf = np.cumsum(p)
        idx.append(torch.from_numpy(np.minimum(np.searchsorted(cdf, rng.random(B) * cdf[-1]), r - 1).astype(np.int64)))
    offs = torch.arange(B, dtype=torch.int64)
    grad = torch.from_numpy(rng.standard_normal((B, T * DIM)).astype(np.float32))

    def one():
        opt.zero_grad(set_to_none=True)
        out = torch.cat([bags[t](idx[t], offs) for t in range(T)], dim=1)
        out.backward(grad)
        opt.step()

    one()
    t0, n = time.perf_counter(), 0
    while time.perf_counter() - t0 < budget_s and n < 50:
        one()
        n += 1
    dt = time.perf_counter() - t0
    return {"value": T * B * n / dt, "unit": "ids/s", "cores": cores,
            "kind": "torch nn.EmbeddingBag(sparse=True) + SparseAdam (stock CPU ops)",
            "sample": f"{n} steps of 26 tables (rows capped at {CPU_SAMPLE_ROW_CAP}) x {CPU_SAMPLE_BATCH} samples"}


def run_reference(args):
    """The reference's CPU implementation of the path: its Ascend kernels have no CPU build, so this arm times
    the CPU restatement of those kernels (oracle/oracle.c, OpenMP over all host cores) on a bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    port, c = _cpu_sample_setup()
    cores = os.cpu_count() or 1
    port.set_num_threads(cores)  # explicit: torchrun exports OMP_NUM_THREADS=1 to its workers
    for i in range(args.warmup):
        _cpu_step(port, c, i + 1)
    t0 = time.perf_counter()
    for i in range(args.steps):
        _cpu_step(port, c, args.warmup + i + 1)
    dt = time.perf_counter() - t0
    ids = c["T"] * c["B"]
    value = ids * args.steps / dt
    sample = (f"each step = 26 tables (rows capped at {CPU_SAMPLE_ROW_CAP}) x {CPU_SAMPLE_BATCH} of the 65536 samples; "
              "oracle C restatement, OpenMP")
    line = {
        "impl": "reference",
        "metric": "embedding ids/sec (fwd+bwd+sparse Adam)", "value": value, "unit": "ids/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "configs[1]: 26 tables dim 128 fp32, one-hot Zipf(1.1), sparse Adam (bounded CPU sample)",
                   "ids_per_step": ids},
        "cpu_baseline": {"value": value, "unit": "ids/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "ids/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


_RESULT_FD = None


def emit(line):
    """The result goes to the process's ORIGINAL stdout as one line; everything else that the run prints
    (library banners such as NCCL's version line included) was redirected to stderr in main()."""
    data = (json.dumps(line) + "\n").encode()
    os.write(_RESULT_FD if _RESULT_FD is not None else 1, data)


def main():
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)  # native libraries write banners to fd 1; keep stdout to the single JSON line
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="step", choices=["step", "ops"],
                    help="step: the benchmark (default).  ops: per-operator measurements of the other entry points")
    ap.add_argument("--no-plan-ahead", action="store_true",
                    help="do not overlap the backward's index work (sort of the row keys, runs, per-row records) "
                         "with the forward on a side stream")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-tables", type=int, default=0,
                    help="reduced case for profiler captures: keep only the K largest tables (1 GPU, no e2e loop)")
    ap.add_argument("--profile-row-cap", type=int, default=524288, help="row cap of the reduced case")
    ap.add_argument("--exchange", default="auto", choices=["auto", "fused", "nccl", "dedup"],
                    help="N>1: dedup (default) = the device-driven dedup exchange: the sample owners fetch the distinct "
                         "rows they need from the table owners and pool locally.  Kept as baselines: pooled rows / "
                         "gradients through NCCL all-to-alls (nccl, the reference's scheme) or stored / loaded inside "
                         "the owners' kernels over peer mappings (fused)")
    ap.add_argument("--fwd-plan", default="ahead", choices=["ahead", "early", "inline"],
                    help="N>1: ahead = the sort-dedup of the next batch's ids runs on a side stream beside the owner phase "
                         "and the fences of the current step (it touches no table); early = the same in a second scratch, "
                         "enqueued right after the forward, so it runs beside the local phase as well; inline = inside "
                         "the forward")
    ap.add_argument("--placement", default="count", choices=["count", "load"],
                    help="N>1: which rank owns which table.  load = balance the distinct rows per table of one profile "
                         "batch (what an owner serves and updates per step); count = equal table counts, big tables apart")
    ap.add_argument("--owner-plan", default="auto", choices=["auto", "ahead", "ahead_main_fence", "inline"],
                    help="N>1: where the owner phase of the exchange makes its plan (sort of the received ids, runs, "
                         "records): ahead = on a side stream beside the local backward phase, after one more fence that "
                         "is issued on that side stream too; ahead_main_fence = the same with the fence on the step's "
                         "stream; inline = inside the owner phase; auto = ahead with more than two ranks, else "
                         "ahead_main_fence")
    ap.add_argument("--cpu-budget", type=float, default=15.0)
    ap.add_argument("--config", default="c2", choices=["c1", "c2", "c3", "c4", "c5"],
                    help="which BASELINE config: c2 (default, the headline: 26-table DLRM step), c1 (one small table, "
                         "Adagrad), c3 (multi-hot, Adagrad), c4 (dynamic hash-keyed table), c5 (row-wise sharded large table)")
    args = ap.parse_args()
    explicit_dedup = args.exchange == "dedup"  # at N = 1: run the exchange kernels on one rank instead of the fused path
    if args.exchange == "auto":
        args.exchange = "dedup"
    if args.workload == "ops":
        run_ops(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        if args.warmup < 3:
            args.warmup = 3
        if args.config in ("c1", "c3"):
            run_tbe_config(args, args.config)
        elif args.config == "c4":
            run_c4(args)
        elif args.config == "c5":
            run_c5(args)
        elif args.exchange == "dedup" and (int(os.environ.get("WORLD_SIZE", "1")) > 1 or explicit_dedup):
            run_dedup_multi(args)
        else:
            run_ours(args)


if __name__ == "__main__":
    main()
