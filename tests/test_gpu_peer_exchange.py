"""Table-wise sharded lookup on 2 GPUs with the pooled rows and gradients moved INSIDE the kernels over peer
mappings (no all-to-all of rows): every rank's pooled buffer and every owner's updated tables must equal, bit for
bit, what the CPU oracle computes for the whole global batch.  Needs two GPUs; skipped otherwise.  One process
per GPU; NVLS is switched off for NCCL and the kernels use plain peer loads / stores."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROWS = [300, 500, 200, 400, 64]
DIMS = [16, 32, 16, 64, 128]
B_LOCAL, L = 24, 2


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, errors):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from oracle import port as orc
        from recsdk_b200.peer import FusedTableWiseExchange
        from recsdk_b200.sharding import TableWiseSharding
        from recsdk_b200.tbe import EmbOptimType, HybridSplitTableBatchedEmbeddingBagsCodegen, PoolingMode

        T = len(ROWS)
        B = world * B_LOCAL
        rng = np.random.default_rng(99)  # identical global data on every rank
        weights = [rng.uniform(-0.1, 0.1, ROWS[t] * DIMS[t]).astype(np.float32) for t in range(T)]
        ids = [rng.integers(0, ROWS[t], size=(B, L)).astype(np.int64) for t in range(T)]
        for t in range(T):
            ids[t][: B // 2] = ids[t][B // 2: B // 2 * 2] % 7  # duplicates across ranks
        grads = [rng.standard_normal((B, DIMS[t])).astype(np.float32) for t in range(T)]

        sh = TableWiseSharding(ROWS, DIMS, world, rank)
        mine = sh.local_tables
        module = HybridSplitTableBatchedEmbeddingBagsCodegen(
            [(ROWS[t], DIMS[t]) for t in mine], optimizer=EmbOptimType.ADAM, pooling_mode=PoolingMode.SUM,
            learning_rate=0.05, eps=1e-8, beta1=0.9, beta2=0.999, device=dev)
        w_local = np.concatenate([weights[t] for t in mine])
        module.weights_dev.data.copy_(torch.from_numpy(w_local))
        fx = FusedTableWiseExchange(sh, B_LOCAL, dev)

        # this rank's samples, fields grouped by owner
        my = slice(rank * B_LOCAL, (rank + 1) * B_LOCAL)
        ids_mine = torch.from_numpy(np.stack([ids[t][my] for t in sh.output_table_order])).to(dev)
        owner_ids = sh.exchange_ids(ids_mine, owner_ordered=True)  # [T_local, B, L]
        assert owner_ids.shape == (len(mine), B, L)
        idx = owner_ids.reshape(-1)
        offs = torch.arange(len(mine) * B + 1, dtype=torch.int64, device=dev) * L

        col = {}
        o = 0
        for t in sh.output_table_order:
            col[t] = o
            o += DIMS[t]
        g_mine = np.zeros((B_LOCAL, sum(DIMS)), np.float32)
        for t in range(T):
            g_mine[:, col[t]:col[t] + DIMS[t]] = grads[t][my]
        fx.grads.local.copy_(torch.from_numpy(g_mine))

        steps = 2
        for it in range(1, steps + 1):
            module.forward_into(idx, offs, out_shards=fx.out_shards)
            fx.fence()
            if it == 1:
                got = fx.pooled.local.cpu().numpy()
                for t in range(T):
                    exp = weights[t].reshape(ROWS[t], DIMS[t])[ids[t][my]]  # [B_local, L, D]
                    acc = np.zeros((B_LOCAL, DIMS[t]), np.float32)
                    for l in range(L):
                        acc = acc + exp[:, l, :]
                    np.testing.assert_array_equal(got[:, col[t]:col[t] + DIMS[t]], acc)
            fx.fence()
            module.backward_from(None, idx, offs, grad_shards=fx.grad_shards)
            fx.fence()

        # oracle over the owner's tables and the global batch
        if mine:
            dims = [DIMS[t] for t in mine]
            wo = np.concatenate([[0], np.cumsum([ROWS[t] * DIMS[t] for t in mine])])[:-1].astype(np.int64)
            do = np.concatenate([[0], np.cumsum(dims)]).astype(np.int32)
            hs = np.concatenate([[0], np.cumsum([ROWS[t] for t in mine])]).astype(np.int64)
            g_owner = np.concatenate([grads[t] for t in mine], axis=1)
            ew, em1, em2 = w_local.copy(), np.zeros_like(w_local), np.zeros_like(w_local)
            idx_np = np.concatenate([ids[t].reshape(-1) for t in mine])
            offs_np = np.arange(len(mine) * B + 1, dtype=np.int64) * L
            for it in range(1, steps + 1):
                orc.tbe_backward(g_owner, ew, em1, em2, wo, do, hs, idx_np, offs_np, len(mine), B, int(do[-1]),
                                 max(dims), 0, 2, 0.05, 1e-8, 0.9, 0.999, it, reduce_chunk=64)
            np.testing.assert_array_equal(module.weights_dev.data.cpu().numpy(), ew)
            np.testing.assert_array_equal(module.momentum1_dev.cpu().numpy(), em1)
            np.testing.assert_array_equal(module.momentum2_dev.cpu().numpy(), em2)
        module.raise_if_error()
        dist.barrier()
        fx.close()
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        errors.put((rank, repr(e)))
        raise


def test_fused_table_wise_exchange_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, errors)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
    for p in procs:
        if p.is_alive():  # pragma: no cover
            p.terminate()
    assert errors.empty(), errors.get()
    assert all(p.exitcode == 0 for p in procs)
