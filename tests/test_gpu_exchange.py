"""The device-driven dedup exchange (recsdk_xchg_*) on ONE GPU: W = 1, 2, 4, 8 logical ranks of one process whose
"peer" buffers are local (the same kernels, plain pointers), bit for bit against the CPU oracle of the sharded
lookup, which restates the two-level summation order (per source rank in index order, then across ranks in
source-rank order -- the reference's deterministic AllUss order).  Row-wise and table-wise placement, SUM / MEAN /
NONE pooling, the three optimizers, ragged / empty / hot bags, and a down-scaled twin of the large row-wise config
(1e6 rows x 64, W = 8, id % W)."""
import numpy as np
import pytest
import torch

from oracle import port

pytestmark = pytest.mark.gpu
DEV = "cuda"

OPT = {1: "EXACT_ADAGRAD", 2: "ADAM", 3: "EXACT_SGD"}


def _make_ranks(rows, dim, world, partition, owner, B, max_ids, opt, mode, acc0=0.0, **kw):
    from recsdk_b200.exchange import DedupExchange, connect_local
    from recsdk_b200.tbe import EmbOptimType, PoolingMode

    ranks = [DedupExchange(rows, dim, world, r, partition=partition, owner=owner, batch_size=B, max_ids=max_ids,
                           optimizer=EmbOptimType[OPT[opt]], pooling_mode=PoolingMode(mode), device=DEV,
                           learning_rate=0.05, eps=1e-8, beta1=0.9, beta2=0.999, initial_accumulator_value=acc0, **kw)
             for r in range(world)]
    if world > 1:
        connect_local(ranks)
    return ranks


def _load(ranks, orc, weights):
    """Same initial tables on the device ranks and in the oracle."""
    for f, w in enumerate(weights):
        orc.load_table(f, w)
    for r, x in enumerate(ranks):
        x.weights_dev.copy_(torch.from_numpy(orc.w[r][:x.weights_dev.numel()]))


def _batches(rng, rows, world, B, max_len, hot=7, one_hot=False):
    F = len(rows)
    out = []
    for q in range(world):
        lens = np.ones(F * B, np.int64) if one_hot else rng.integers(0, max_len + 1, size=F * B)
        idx = np.concatenate([rng.integers(0, rows[i // B], size=lens[i]) % (hot if i % 3 == 0 else rows[i // B])
                              for i in range(F * B)] + [np.empty(0, np.int64)]).astype(np.int64)
        offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        out.append((idx, offs))
    return out


def _run_and_compare(ranks, orc, batches, grads, B, mode, steps=2, plan_ahead=False, fwd_plan_ahead=False,
                     fwd_plan_early=False):
    world = len(ranks)
    dev_b = [(torch.from_numpy(i).to(DEV), torch.from_numpy(o).to(DEV)) for i, o in batches]
    dev_g = [torch.from_numpy(g).to(DEV) for g in grads]
    for step_no in range(steps):
        exp_out = orc.step(batches, grads, B, mode)
        outs = [ranks[q].forward(*dev_b[q]) for q in range(world)]  # phase by phase, all ranks: the stream orders them
        if plan_ahead:  # every rank's ids are in the inboxes: the owners' index work goes to their side streams
            for q in range(world):
                ranks[q].plan_owner_ahead()
        if fwd_plan_early and step_no + 1 < steps:  # double-buffered scratch: the next plan beside the local phase already
            for q in range(world):
                ranks[q].plan_forward_ahead(*dev_b[q])
        for q in range(world):
            ranks[q].backward_local(dev_g[q])
        if fwd_plan_ahead and step_no + 1 < steps:  # the next step's sort-dedup, beside this step's owner phase
            for q in range(world):
                ranks[q].plan_forward_ahead(*dev_b[q])
        for q in range(world):
            ranks[q].backward_owner()
        for q in range(world):
            np.testing.assert_array_equal(outs[q].cpu().numpy(), exp_out[q])
    for r, x in enumerate(ranks):
        x.raise_if_error()
        n = x.weights_dev.numel()
        np.testing.assert_array_equal(x.weights_dev.cpu().numpy(), orc.w[r][:n])
        if x.momentum1_dev is not None:
            np.testing.assert_array_equal(x.momentum1_dev.cpu().numpy(), orc.m1[r][:n])
        if x.momentum2_dev is not None:
            np.testing.assert_array_equal(x.momentum2_dev.cpu().numpy(), orc.m2[r][:n])


ROWS = [1000, 37, 5000, 64]


@pytest.mark.parametrize("opt", [1, 2, 3])
@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("partition", ["row", "table"])
def test_exchange_loopback_bit_exact(partition, world, mode, opt):
    rng = np.random.default_rng(1000 + 17 * world + mode)
    F, D, B, max_len = len(ROWS), 32, 24, 3
    owner = [f % world for f in range(F)] if partition == "table" else None
    max_ids = F * B * max_len
    # every id of a rank may go to one owner in this small case: inbox sized for it
    ranks = _make_ranks(ROWS, D, world, partition, owner, B, max_ids, opt, mode, acc0=0.1 if opt == 1 else 0.0,
                        inbox_cap=max_ids)
    orc = port.ShardedDedupOracle(ROWS, D, world, partition, owner, optimizer=opt, lr=0.05, eps=1e-8,
                                  initial_accumulator_value=0.1 if opt == 1 else 0.0)
    _load(ranks, orc, [rng.uniform(-0.1, 0.1, (r, D)).astype(np.float32) for r in ROWS])
    batches = _batches(rng, ROWS, world, B, max_len)
    grads = [rng.standard_normal((b[0].size, D) if mode == 2 else (B, F * D)).astype(np.float32) for b in batches]
    _run_and_compare(ranks, orc, batches, grads, B, mode)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("partition", ["row", "table"])
def test_exchange_one_id_per_bag_path_bit_exact(partition, world, mode):
    """The caller states one id per bag: every fetched row is stored straight to the bags of its run (short runs and
    chunks of long runs).  Hot rows give runs far beyond the chunk length."""
    rng = np.random.default_rng(400 + world)
    rows, D, B = [300, 2000, 17], 64, 500
    F = len(rows)
    owner = [f % world for f in range(F)] if partition == "table" else None
    ranks = _make_ranks(rows, D, world, partition, owner, B, F * B, 2, mode, inbox_cap=F * B, one_hot=True)
    orc = port.ShardedDedupOracle(rows, D, world, partition, owner, optimizer=2, lr=0.05)
    _load(ranks, orc, [rng.uniform(-0.1, 0.1, (r, D)).astype(np.float32) for r in rows])
    batches = _batches(rng, rows, world, B, 1, hot=2, one_hot=True)
    grads = [rng.standard_normal((B, F * D)).astype(np.float32) for _ in batches]
    _run_and_compare(ranks, orc, batches, grads, B, mode)
    assert ranks[0].counters()[3] > 0


def test_exchange_one_id_per_bag_promise_is_checked():
    rng = np.random.default_rng(3)
    rows, D, B = [100], 8, 16
    ranks = _make_ranks(rows, D, 1, "row", None, B, 3 * B, 3, 0, inbox_cap=3 * B, one_hot=True)
    lens = np.full(B, 1, np.int64)
    lens[5], lens[9] = 2, 0  # still B ids in total, but not one per bag: only the device can see it
    idx = torch.from_numpy(rng.integers(0, 100, int(lens.sum())).astype(np.int64)).to(DEV)
    offs = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)).to(DEV)
    ranks[0].forward(idx, offs)
    with pytest.raises(RuntimeError):
        ranks[0].raise_if_error()
    lens[9] = 1  # one id too many: rejected on the host
    idx = torch.from_numpy(rng.integers(0, 100, int(lens.sum())).astype(np.int64)).to(DEV)
    offs = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)).to(DEV)
    with pytest.raises(RuntimeError):
        ranks[0].forward(idx, offs)


@pytest.mark.parametrize("partition", ["row", "table"])
def test_exchange_owner_plan_on_side_stream_bit_exact(partition):
    """The owner phase split in two: its index work on a side stream while the local phase runs, the row update after
    the gradient sums have arrived.  Same bits."""
    rng = np.random.default_rng(31)
    F, D, B, world = len(ROWS), 32, 40, 4
    owner = [f % world for f in range(F)] if partition == "table" else None
    ranks = _make_ranks(ROWS, D, world, partition, owner, B, F * B * 3, 2, 0, inbox_cap=F * B * 3)
    orc = port.ShardedDedupOracle(ROWS, D, world, partition, owner, optimizer=2, lr=0.05)
    _load(ranks, orc, [rng.uniform(-0.1, 0.1, (r, D)).astype(np.float32) for r in ROWS])
    batches = _batches(rng, ROWS, world, B, 3)
    grads = [rng.standard_normal((B, F * D)).astype(np.float32) for _ in batches]
    _run_and_compare(ranks, orc, batches, grads, B, 0, steps=3, plan_ahead=True)


@pytest.mark.parametrize("mode", [0, 2])
def test_exchange_forward_plan_ahead_bit_exact(mode):
    """The forward split in two: the sort-dedup of the next step's ids on a side stream while the owner phase of the
    current step runs (it touches no table), the fetch after it.  Same bits; a plan made for other tensors is refused."""
    rng = np.random.default_rng(33)
    F, D, B, world = len(ROWS), 32, 40, 4
    ranks = _make_ranks(ROWS, D, world, "row", None, B, F * B * 3, 2, mode, inbox_cap=F * B * 3)
    orc = port.ShardedDedupOracle(ROWS, D, world, "row", optimizer=2, lr=0.05)
    _load(ranks, orc, [rng.uniform(-0.1, 0.1, (r, D)).astype(np.float32) for r in ROWS])
    batches = _batches(rng, ROWS, world, B, 3)
    grads = [rng.standard_normal((b[0].size, D) if mode == 2 else (B, F * D)).astype(np.float32) for b in batches]
    _run_and_compare(ranks, orc, batches, grads, B, mode, steps=3, plan_ahead=True, fwd_plan_ahead=True)
    # the same with a second scratch per rank: the next plan is made right after the forward, beside the local phase
    ranks2 = _make_ranks(ROWS, D, world, "row", None, B, F * B * 3, 2, mode, inbox_cap=F * B * 3, double_buffer=True)
    orc2 = port.ShardedDedupOracle(ROWS, D, world, "row", optimizer=2, lr=0.05)
    rng2 = np.random.default_rng(33)
    _load(ranks2, orc2, [rng2.uniform(-0.1, 0.1, (r, D)).astype(np.float32) for r in ROWS])
    _run_and_compare(ranks2, orc2, batches, grads, B, mode, steps=4, plan_ahead=True, fwd_plan_early=True)
    idx, offs = (torch.from_numpy(a).to(DEV) for a in batches[0])
    ranks[0].plan_forward_ahead(idx, offs)
    with pytest.raises(RuntimeError, match="other indices"):
        ranks[0].forward(idx.clone(), offs)


def test_exchange_hot_rows_long_runs_and_wide_rows():
    """Runs far longer than the chunk length on the requesting ranks (chunk sums) and rows of 128 floats."""
    rng = np.random.default_rng(5)
    rows, D, B, world = [40, 3000], 128, 400, 4
    owner = [0, 2]
    ranks = _make_ranks(rows, D, world, "table", owner, B, 2 * B * 3, 2, 0, inbox_cap=2 * B * 3)
    orc = port.ShardedDedupOracle(rows, D, world, "table", owner, optimizer=2, lr=0.05)
    _load(ranks, orc, [rng.uniform(-0.1, 0.1, (r, D)).astype(np.float32) for r in rows])
    batches = _batches(rng, rows, world, B, 3, hot=3)
    grads = [rng.standard_normal((B, 2 * D)).astype(np.float32) for _ in batches]
    _run_and_compare(ranks, orc, batches, grads, B, 0)
    assert ranks[0].counters()[3] > 0  # some ids lived in chunked runs


def test_exchange_fetch_repeated_on_one_plan():
    """A fetch may be repeated on the plan it belongs to: the records of the local backward phase, which the fetch
    writes, reserve their chunk slots from zero every time.  One id per bag, hot rows (chunked runs)."""
    import ctypes as C

    from recsdk_b200 import _lib
    from recsdk_b200.ops import _stream, check

    rng = np.random.default_rng(8)
    rows, D, B, world = [40, 3000], 128, 1200, 2
    ranks = _make_ranks(rows, D, world, "table", [0, 1], B, 2 * B, 2, 0, inbox_cap=2 * B, one_hot=True)
    orc = port.ShardedDedupOracle(rows, D, world, "table", [0, 1], optimizer=2, lr=0.05)
    _load(ranks, orc, [rng.uniform(-0.1, 0.1, (r, D)).astype(np.float32) for r in rows])
    batches = _batches(rng, rows, world, B, 1, hot=3, one_hot=True)
    grads = [rng.standard_normal((B, 2 * D)).astype(np.float32) for _ in batches]
    exp_out = orc.step(batches, grads, B, 0)
    dev_b = [(torch.from_numpy(i).to(DEV), torch.from_numpy(o).to(DEV)) for i, o in batches]
    outs = [ranks[q].forward(*dev_b[q]) for q in range(world)]
    for q in range(world):
        x, (idx, offs) = ranks[q], dev_b[q]
        again = torch.empty_like(outs[q])
        for _ in range(4):
            check(_lib.load().recsdk_xchg_forward(C.byref(x._x), idx.data_ptr(), offs.data_ptr(), idx.numel(), 0,
                                                  again.data_ptr(), 2, _stream()), "recsdk_xchg_forward")
        np.testing.assert_array_equal(again.cpu().numpy(), exp_out[q])
        np.testing.assert_array_equal(outs[q].cpu().numpy(), exp_out[q])
    for q in range(world):
        ranks[q].backward_local(torch.from_numpy(grads[q]).to(DEV))
    for q in range(world):
        ranks[q].backward_owner()
    for r, x in enumerate(ranks):
        x.raise_if_error()
        assert x.counters()[3] > 0  # chunked runs were there
        n = x.weights_dev.numel()
        np.testing.assert_array_equal(x.weights_dev.cpu().numpy(), orc.w[r][:n])
        np.testing.assert_array_equal(x.momentum2_dev.cpu().numpy(), orc.m2[r][:n])


def test_exchange_large_rowwise_twin():
    """Down-scaled twin of the large row-wise config: one table of 1e6 rows x 64, W = 8, rows placed by id % W,
    one-hot Zipf(1.05) ids, Adam; 4096 ids per rank."""
    from tests.golden.driver import zipf_ids

    rng = np.random.default_rng(55)
    rows, D, B, world = [1_000_000], 64, 4096, 8
    ranks = _make_ranks(rows, D, world, "row", None, B, B, 2, 0)
    orc = port.ShardedDedupOracle(rows, D, world, "row", optimizer=2, lr=0.05)
    _load(ranks, orc, [rng.uniform(-0.05, 0.05, (rows[0], D)).astype(np.float32)])
    perm_a, perm_b = 7919, 104729  # rank -> id by an affine map so that hot rows spread over the ranks
    batches = []
    for q in range(world):
        ids = (zipf_ids(rng, B, rows[0], 1.05) * perm_a + perm_b) % rows[0]
        batches.append((ids.astype(np.int64), np.arange(B + 1, dtype=np.int64)))
    grads = [rng.standard_normal((B, D)).astype(np.float32) for _ in batches]
    _run_and_compare(ranks, orc, batches, grads, B, 0, steps=2)


def test_exchange_inbox_overflow_sets_status():
    rng = np.random.default_rng(2)
    rows, D, B, world = [1000], 8, 64, 2
    ranks = _make_ranks(rows, D, world, "row", None, B, B, 3, 0, inbox_cap=4)
    idx = torch.from_numpy(rng.permutation(1000)[:B].astype(np.int64)).to(DEV)
    offs = torch.arange(B + 1, dtype=torch.int64, device=DEV)
    ranks[0].forward(idx, offs)
    with pytest.raises(RuntimeError):
        ranks[0].raise_if_error()
