"""Dedup-exchange lookups -- row-wise (rows split by id % W) and table-wise (whole tables on ranks, distinct rows
fetched by the sample owners) -- on 2 GPUs against the CPU oracle run on the whole tables and the global batch.  The forward pools the same rows in the same order -> bit-exact.  The backward sums a row's gradients
in two levels (per source rank, then across ranks in rank order) where the single-table oracle sums them flat, so
the updated tables are compared at 1e-5; running the step twice from the same state must give identical bits.
Needs two GPUs; skipped otherwise."""
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


def _worker(rank, world, port, errors, scheme="row"):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from oracle import port as orc
        from recsdk_b200.rowwise import RowWiseShardedEmbeddingBag, TableWiseDedupEmbeddingBag
        from recsdk_b200.tbe import EmbOptimType, PoolingMode

        F, D = len(ROWS), DIM
        B = world * B_LOCAL
        owner = [f % world for f in range(F)]
        rng = np.random.default_rng(321)  # identical global data on every rank
        weights = [rng.uniform(-0.1, 0.1, (ROWS[f], D)).astype(np.float32) for f in range(F)]
        lens = rng.integers(0, MAX_L + 1, size=(F, B))
        ids = [[rng.integers(0, ROWS[f], size=lens[f, b]).astype(np.int64) % (7 if b % 3 == 0 else ROWS[f])
                for b in range(B)] for f in range(F)]
        grad = rng.standard_normal((B, F * D)).astype(np.float32)

        def csr(sample_range):
            idx = np.concatenate([ids[f][b] for f in range(F) for b in sample_range] + [np.empty(0, np.int64)])
            ln = np.array([lens[f, b] for f in range(F) for b in sample_range], np.int64)
            return idx.astype(np.int64), np.concatenate([[0], np.cumsum(ln)]).astype(np.int64)

        kw = dict(optimizer=EmbOptimType.ADAM, pooling_mode=PoolingMode.SUM, device=dev, learning_rate=0.05, eps=1e-8,
                  beta1=0.9, beta2=0.999)
        if scheme == "row":
            bag = RowWiseShardedEmbeddingBag(ROWS, D, world, rank, **kw)
            mine_tables = list(range(F))
            shard_of = lambda a: a[rank::world]  # noqa: E731
        else:
            bag = TableWiseDedupEmbeddingBag(ROWS, D, owner, world, rank, **kw)
            if scheme == "table_pull":  # rows and gradient rows pulled out of peer-mapped buffers instead of all-to-alls
                bag.enable_peer_pull(B_LOCAL * MAX_L)
            mine_tables = [f for f in range(F) if owner[f] == rank]
            shard_of = lambda a: a  # noqa: E731
        for f in mine_tables:
            shard = shard_of(weights[f])
            bag.local_table(f)[:shard.shape[0]].copy_(torch.from_numpy(shard))
        mine = range(rank * B_LOCAL, (rank + 1) * B_LOCAL)
        idx_l, offs_l = csr(mine)
        idx_t, offs_t = torch.from_numpy(idx_l).to(dev), torch.from_numpy(offs_l).to(dev)
        g_t = torch.from_numpy(grad[rank * B_LOCAL:(rank + 1) * B_LOCAL].copy()).to(dev)

        # oracle on the whole tables, global batch
        idx_g, offs_g = csr(range(B))
        w_flat = np.concatenate([w.reshape(-1) for w in weights])
        wo = np.concatenate([[0], np.cumsum([ROWS[f] * D for f in range(F)])])[:-1].astype(np.int64)
        do = (np.arange(F + 1) * D).astype(np.int32)
        hs = np.concatenate([[0], np.cumsum(ROWS)]).astype(np.int64)
        exp_out = orc.tbe_forward(w_flat, wo, do, idx_g, offs_g, F, B, F * D, D, 0)
        ew, em1, em2 = w_flat.copy(), np.zeros_like(w_flat), np.zeros_like(w_flat)

        state0 = [t.clone() for t in (bag.owner.weights_dev.data, bag.owner.momentum1_dev, bag.owner.momentum2_dev)]
        results = []
        for attempt in range(2):
            for t, s0 in zip((bag.owner.weights_dev.data, bag.owner.momentum1_dev, bag.owner.momentum2_dev), state0):
                t.copy_(s0)
            bag.owner.iter[0] = 0
            for it in (1, 2):
                out = bag.forward(idx_t, offs_t)
                if attempt == 0 and it == 1:
                    np.testing.assert_array_equal(out.cpu().numpy(), exp_out[rank * B_LOCAL:(rank + 1) * B_LOCAL])
                bag.backward(g_t)
            results.append({f: bag.local_table(f).clone() for f in mine_tables})
        for f in mine_tables:
            assert torch.equal(results[0][f], results[1][f])  # run-to-run identical bits
        for it in (1, 2):
            orc.tbe_backward(grad, ew, em1, em2, wo, do, hs, idx_g, offs_g, F, B, F * D, D, 0, 2, 0.05, 1e-8, 0.9,
                             0.999, it, reduce_chunk=64)
        for f in mine_tables:
            exp = shard_of(ew[wo[f]:wo[f] + ROWS[f] * D].reshape(ROWS[f], D))
            got = results[0][f][:exp.shape[0]].cpu().numpy()
            np.testing.assert_allclose(got, exp, rtol=0, atol=1e-5)
        dist.barrier()
        if scheme == "table_pull":
            bag.close()
            dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        errors.put((rank, repr(e)))
        raise


@pytest.mark.parametrize("scheme", ["row", "table", "table_pull"])
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
        p.join(90)
    for p in procs:
        if p.is_alive():  # pragma: no cover
            p.terminate()
    assert errors.empty(), errors.get()
    assert all(p.exitcode == 0 for p in procs)


@pytest.mark.parametrize("scheme", ["row", "table"])
def test_dedup_exchange_single_rank_is_bit_exact(scheme):
    """World 1: the same code path without a process group; both summation levels collapse to the oracle's order."""
    from oracle import port as orc
    from recsdk_b200.rowwise import RowWiseShardedEmbeddingBag, TableWiseDedupEmbeddingBag
    from recsdk_b200.tbe import EmbOptimType, PoolingMode

    F, D, B = len(ROWS), DIM, 40
    rng = np.random.default_rng(5)
    weights = [rng.uniform(-0.1, 0.1, (ROWS[f], D)).astype(np.float32) for f in range(F)]
    lens = rng.integers(0, MAX_L + 1, size=F * B)
    idx = np.concatenate([rng.integers(0, ROWS[i // B], size=lens[i]) % (5 if i % 4 == 0 else ROWS[i // B])
                          for i in range(F * B)]).astype(np.int64)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    grad = rng.standard_normal((B, F * D)).astype(np.float32)
    for mode in (PoolingMode.SUM, PoolingMode.MEAN):
        kw = dict(optimizer=EmbOptimType.EXACT_ADAGRAD, pooling_mode=mode, device="cuda", learning_rate=0.05, eps=1e-8,
                  initial_accumulator_value=0.1)
        bag = (RowWiseShardedEmbeddingBag(ROWS, D, 1, 0, **kw) if scheme == "row"
               else TableWiseDedupEmbeddingBag(ROWS, D, [0] * F, 1, 0, **kw))
        for f in range(F):
            bag.local_table(f).copy_(torch.from_numpy(weights[f]))
        w_flat = np.concatenate([w.reshape(-1) for w in weights])
        wo = np.concatenate([[0], np.cumsum([ROWS[f] * D for f in range(F)])])[:-1].astype(np.int64)
        do = (np.arange(F + 1) * D).astype(np.int32)
        hs = np.concatenate([[0], np.cumsum(ROWS)]).astype(np.int64)
        ew, em1 = w_flat.copy(), np.full_like(w_flat, 0.1)
        for it in (1, 2):
            exp_out = orc.tbe_forward(ew, wo, do, idx, offs, F, B, F * D, D, int(mode))
            out = bag.forward(torch.from_numpy(idx).cuda(), torch.from_numpy(offs).cuda())
            np.testing.assert_array_equal(out.cpu().numpy(), exp_out)
            bag.backward(torch.from_numpy(grad).cuda())
            orc.tbe_backward(grad, ew, em1, None, wo, do, hs, idx, offs, F, B, F * D, D, int(mode), 1, 0.05, 1e-8,
                             reduce_chunk=64)
        got = np.concatenate([bag.local_table(f).cpu().numpy().reshape(-1) for f in range(F)])
        np.testing.assert_array_equal(got, ew)
