"""CPU checks of the sharded-lookup oracle itself (oracle/port.py:ShardedDedupOracle): its two-level summation is a
re-association of the flat single-process lookup, and its placement helpers round-trip."""
import numpy as np
import pytest

from oracle import port


def _batches(rng, rows, world, B, max_len, hot=7):
    F = len(rows)
    out = []
    for q in range(world):
        lens = rng.integers(0, max_len + 1, size=F * B)
        idx = np.concatenate([rng.integers(0, rows[i // B], size=lens[i]) % (hot if i % 3 == 0 else rows[i // B])
                              for i in range(F * B)] + [np.empty(0, np.int64)]).astype(np.int64)
        offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        out.append((idx, offs))
    return out


@pytest.mark.parametrize("partition", ["row", "table"])
def test_exchange_matches_flat_lookup_semantics(partition):
    """The two-level order is a re-association only: against the flat single-process oracle (one sum per row over
    the global batch) the updated tables agree to 1e-5, the forward bit for bit."""
    rng = np.random.default_rng(9)
    rows, D, B, world, F = [500, 80], 16, 32, 4, 2
    weights = [rng.uniform(-0.1, 0.1, (r, D)).astype(np.float32) for r in rows]
    orc = port.ShardedDedupOracle(rows, D, world, partition, owner=[1, 3], optimizer=2, lr=0.05)
    for f, w in enumerate(weights):
        orc.load_table(f, w)
    batches = _batches(rng, rows, world, B, 4)
    grads = [rng.standard_normal((B, F * D)).astype(np.float32) for _ in batches]
    outs = orc.step(batches, grads, B, 0)
    # global batch, feature-major over all ranks' samples
    Bg = world * B
    idx_g, lens_g = [], []
    for f in range(F):
        for q in range(world):
            i, o = batches[q]
            idx_g.append(i[o[f * B]:o[(f + 1) * B]])
            lens_g.append(np.diff(o[f * B:(f + 1) * B + 1]))
    idx_g = np.concatenate(idx_g).astype(np.int64)
    offs_g = np.concatenate([[0], np.cumsum(np.concatenate(lens_g))]).astype(np.int64)
    w_flat = np.concatenate([w.reshape(-1) for w in weights])
    wo = np.array([0, rows[0] * D], np.int64)
    do = (np.arange(F + 1) * D).astype(np.int32)
    hs = np.array([0, rows[0], rows[0] + rows[1]], np.int64)
    exp_out = port.tbe_forward(w_flat, wo, do, idx_g, offs_g, F, Bg, F * D, D, 0)
    np.testing.assert_array_equal(np.concatenate(outs), exp_out)
    m1, m2 = np.zeros_like(w_flat), np.zeros_like(w_flat)
    port.tbe_backward(np.concatenate(grads), w_flat, m1, m2, wo, do, hs, idx_g, offs_g, F, Bg, F * D, D, 0, 2, 0.05, 1e-8,
                      0.9, 0.999, 1, reduce_chunk=64)
    got = np.concatenate([orc.table(f).reshape(-1) for f in range(F)])
    np.testing.assert_allclose(got, w_flat, rtol=0, atol=1e-5)


def test_oracle_placement_round_trip():
    rng = np.random.default_rng(1)
    rows, D = [101, 7, 64], 4
    for partition, owner in (("row", None), ("table", [2, 0, 2])):
        orc = port.ShardedDedupOracle(rows, D, 3, partition, owner=owner)
        ws = [rng.standard_normal((r, D)).astype(np.float32) for r in rows]
        for f, w in enumerate(ws):
            orc.load_table(f, w)
        for f, w in enumerate(ws):
            np.testing.assert_array_equal(orc.table(f), w)


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_exchange_layouts_agree_with_the_oracle_placement(world):
    """Host-side layout of the exchange (linear row numbering, per-rank bases) against the oracle's own placement:
    row `idx` of table f must land on the same rank at the same local row in both."""
    from recsdk_b200.exchange import row_wise_layout, table_wise_layout

    rng = np.random.default_rng(world)
    rows = [int(r) for r in rng.integers(1, 2000, size=7)]
    owner = [int(o) for o in rng.integers(0, world, size=7)]
    orc_t = port.ShardedDedupOracle(rows, 4, world, "table", owner=owner)
    part_base, rank_base = table_wise_layout(rows, owner, world)
    assert rank_base[0] == 0 and rank_base[world] == sum(rows)
    for f, r in enumerate(rows):
        idx = rng.integers(0, r, size=20)
        own, lrow = orc_t.place(f, idx)
        lin = part_base[f] + idx
        np.testing.assert_array_equal(np.searchsorted(np.array(rank_base[1:]), lin, side="right"), own)
        np.testing.assert_array_equal(lin - np.array(rank_base)[own], lrow)
    orc_r = port.ShardedDedupOracle(rows, 4, world, "row")
    part_base, rank_base, local = row_wise_layout(rows, world)
    assert rank_base[world] == sum(sum(x) for x in local)
    for f, r in enumerate(rows):
        idx = rng.integers(0, r, size=20)
        own, lrow = orc_r.place(f, idx)
        np.testing.assert_array_equal(idx % world, own)
        lin = np.array([part_base[int(o) * len(rows) + f] for o in own]) + idx // world
        np.testing.assert_array_equal(lin - np.array(rank_base)[own], lrow)
        assert (lin < np.array(rank_base)[own + 1]).all()
