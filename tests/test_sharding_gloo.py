"""The table-wise exchange plan (ids out, pooled rows back, gradients out) over world_size-2 and -3 gloo groups
on CPU: every rank must end up with exactly the values a single process would compute."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROWS = [1000, 50, 700, 20, 300]
DIMS = [8, 4, 8, 16, 4]
B, L = 6, 2


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _ident(t, s, b, l):
    return ((t * 100 + s) * 100 + b) * 10 + l


def _worker(rank, world, port, errors):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from recsdk_b200.sharding import TableWiseSharding, greedy_table_placement

        T = len(ROWS)
        sh = TableWiseSharding(ROWS, DIMS, world, rank)
        assert sh.owner == greedy_table_placement(ROWS, DIMS, world)
        assert sorted(sh.output_table_order) == list(range(T))
        # ids: value encodes (table, source rank, sample, position)
        ids = torch.tensor([[[_ident(t, rank, b, l) for l in range(L)] for b in range(B)] for t in range(T)])
        got = sh.exchange_ids(ids)
        assert got.shape == (len(sh.local_tables), world * B, L)
        for i, t in enumerate(sh.local_tables):
            for s in range(world):
                for b in range(B):
                    for l in range(L):
                        assert int(got[i, s * B + b, l]) == _ident(t, s, b, l)
        # pooled outputs of the owner: element (sample s*B+b, table t, column d) = t*1e4 + s*1e3 + b*10 + d/100
        cols = []
        for t in sh.local_tables:
            d = torch.arange(DIMS[t], dtype=torch.float32) / 100
            sb = torch.tensor([[s * 1000 + b * 10 for b in range(B)] for s in range(world)], dtype=torch.float32).view(-1, 1)
            cols.append(t * 10000 + sb + d)
        pooled = torch.cat(cols, dim=1) if cols else torch.empty(world * B, 0)
        out = sh.exchange_outputs(pooled, B)
        assert out.shape == (B, sum(DIMS))
        o = 0
        for t in sh.output_table_order:
            exp = t * 10000 + rank * 1000 + torch.arange(B, dtype=torch.float32).view(-1, 1) * 10 + \
                torch.arange(DIMS[t], dtype=torch.float32) / 100
            assert torch.equal(out[:, o:o + DIMS[t]], exp), (rank, t)
            o += DIMS[t]
        # gradients travel the transposed way and land where the pooled rows came from
        back = sh.exchange_gradients(out)
        assert torch.equal(back, pooled)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        errors.put((rank, repr(e)))
        raise


@pytest.mark.parametrize("world", [2, 3])
def test_table_wise_exchanges(world):
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, errors)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert errors.empty(), errors.get()
    assert all(p.exitcode == 0 for p in procs)


def test_single_rank_is_identity():
    from recsdk_b200.sharding import TableWiseSharding

    sh = TableWiseSharding(ROWS, DIMS, 1, 0)
    ids = torch.arange(len(ROWS) * B * L).view(len(ROWS), B, L)
    assert torch.equal(sh.exchange_ids(ids), ids)
    x = torch.randn(B, sum(DIMS))
    assert torch.equal(sh.exchange_outputs(x, B), x)
    assert torch.equal(sh.exchange_gradients(x), x)


def test_placement_by_load_balances_load_under_a_byte_cap():
    from recsdk_b200.sharding import greedy_table_placement

    rows = [4000, 10, 3000, 20, 2000, 30, 1000, 40]
    dims = [8] * 8
    loads = [5, 100, 5, 90, 5, 80, 5, 70]  # the small tables are the busy ones
    by_count = greedy_table_placement(rows, dims, 2)
    assert sorted(by_count.count(r) for r in range(2)) == [4, 4]
    by_load = greedy_table_placement(rows, dims, 2, loads=loads)
    work = [sum(loads[t] for t in range(8) if by_load[t] == r) for r in range(2)]
    assert abs(work[0] - work[1]) <= 10 and by_load == greedy_table_placement(rows, dims, 2, loads=loads)
    # a cap that only lets one of the big tables on a rank
    cap = (4000 + 1000 + 100) * 8 * 12
    capped = greedy_table_placement(rows, dims, 2, loads=[1] * 8, bytes_cap=cap)
    size = [sum(rows[t] * 8 * 12 for t in range(8) if capped[t] == r) for r in range(2)]
    assert capped[0] != capped[2] and max(size) <= (4000 + 2000 + 100) * 8 * 12
    with pytest.raises(ValueError):
        greedy_table_placement(rows, dims, 2, loads=[1, 2])
