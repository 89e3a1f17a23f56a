"""The dedup-exchange lookups -- row-wise (rows split by id % W) and table-wise (whole tables on ranks, distinct rows
fetched by the sample owners) -- as one process per GPU on 2 GPUs, with the peers' tables and inboxes mapped by CUDA
IPC and NCCL one-element all-reduces as fences.  Forward, updated tables and optimizer state are compared bit for
bit with the CPU oracle of the sharded lookup (two-level summation order).  Needs two GPUs; skipped otherwise (the
same kernels run as logical ranks on one GPU in test_gpu_exchange.py)."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROWS = [1000, 37, 5000]
DIM = 32
B_LOCAL, MAX_L = 48, 3


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, errors, scheme):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from oracle import port as orc_port
        from recsdk_b200.rowwise import RowWiseShardedEmbeddingBag, TableWiseDedupEmbeddingBag
        from recsdk_b200.tbe import EmbOptimType, PoolingMode

        F, D = len(ROWS), DIM
        owner = [f % world for f in range(F)]
        rng = np.random.default_rng(321)  # identical global data on every rank
        weights = [rng.uniform(-0.1, 0.1, (ROWS[f], D)).astype(np.float32) for f in range(F)]
        batches, grads = [], []
        for q in range(world):
            lens = rng.integers(0, MAX_L + 1, size=F * B_LOCAL)
            idx = np.concatenate([rng.integers(0, ROWS[i // B_LOCAL], size=lens[i]) % (7 if i % 3 == 0 else ROWS[i // B_LOCAL])
                                  for i in range(F * B_LOCAL)] + [np.empty(0, np.int64)]).astype(np.int64)
            batches.append((idx, np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)))
            grads.append(rng.standard_normal((B_LOCAL, F * D)).astype(np.float32))
        kw = dict(optimizer=EmbOptimType.ADAM, pooling_mode=PoolingMode.SUM, device=dev, learning_rate=0.05, eps=1e-8,
                  beta1=0.9, beta2=0.999, batch_size=B_LOCAL, max_ids=F * B_LOCAL * MAX_L, inbox_cap=F * B_LOCAL * MAX_L)
        if scheme == "row":
            bag = RowWiseShardedEmbeddingBag(ROWS, D, world, rank, **kw)
            orc = orc_port.ShardedDedupOracle(ROWS, D, world, "row", optimizer=2, lr=0.05)
        else:
            bag = TableWiseDedupEmbeddingBag(ROWS, D, owner, world, rank, **kw)
            orc = orc_port.ShardedDedupOracle(ROWS, D, world, "table", owner=owner, optimizer=2, lr=0.05)
        for f, w in enumerate(weights):
            orc.load_table(f, w)
        bag.weights_dev.copy_(torch.from_numpy(orc.w[rank][:bag.weights_dev.numel()]))
        idx_t, offs_t = (torch.from_numpy(a).to(dev) for a in batches[rank])
        g_t = torch.from_numpy(grads[rank]).to(dev)
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(2):
            exp = orc.step(batches, grads, B_LOCAL, 0)
            out = bag.forward(idx_t, offs_t)
            bag.backward(g_t, plan_ahead=(scheme == "row"))  # [fence, owner plan ahead ->] local sums -> fence -> owner update -> fence
            np.testing.assert_array_equal(out.cpu().numpy(), exp[rank])
        bag.raise_if_error()
        n = bag.weights_dev.numel()
        np.testing.assert_array_equal(bag.weights_dev.cpu().numpy(), orc.w[rank][:n])
        np.testing.assert_array_equal(bag.momentum1_dev.cpu().numpy(), orc.m1[rank][:n])
        np.testing.assert_array_equal(bag.momentum2_dev.cpu().numpy(), orc.m2[rank][:n])
        dist.barrier()
        bag.close()
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        errors.put((rank, repr(e)))
        raise


@pytest.mark.parametrize("scheme", ["row", "table"])
def test_dedup_exchange_lookup_two_gpus(scheme):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, errors, scheme)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    for p in procs:
        if p.is_alive():  # pragma: no cover
            p.terminate()
    assert errors.empty(), errors.get()
    assert all(p.exitcode == 0 for p in procs)
