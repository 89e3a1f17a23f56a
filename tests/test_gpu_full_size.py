"""The benchmark configs at FULL size on one GPU, checked through properties that do not need the CPU oracle to
walk 20 M indices: a second, independent device computation of the same quantity with stock torch ops
(`embedding_bag`, `index_add_`, elementwise optimizer formulas), run-to-run bit identity, and untouched rows.

Tolerances: the forward adds rows in index order on both sides -> compared at 1e-6 relative; the torch reference
of the backward sums gradient rows with float atomics in arbitrary order, ours in a fixed order -> 2e-4
(relative to the largest magnitude of the tensor), the gate of the reference's own operator test being 1e-4 on
4 epochs of a small case."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _tables(seed, n, lo, hi):
    from recsdk_b200.synthetic import table_rows_log_uniform

    return table_rows_log_uniform(seed, n, lo, hi)


def _module(rows, D, opt, mode, lr=0.01, acc0=0.0):
    from recsdk_b200.tbe import HybridSplitTableBatchedEmbeddingBagsCodegen

    return HybridSplitTableBatchedEmbeddingBagsCodegen(
        [(r, D) for r in rows], optimizer=opt, pooling_mode=mode, learning_rate=lr, eps=1e-8, beta1=0.9, beta2=0.999,
        device=torch.device(DEV), weights_init=(-0.05, 0.05), seed=3, initial_accumulator_value=acc0,
        bounds_check=True)


def _per_table(idx, offs, T, B):
    """(indices_t, offsets_t relative) of every table from the feature-major CSR."""
    out = []
    for t in range(T):
        o = offs[t * B:(t + 1) * B + 1]
        s, e = int(o[0].item()), int(o[-1].item())
        out.append((idx[s:e], o[:-1] - s))
    return out


def test_multi_hot_config_full_size_forward_and_adagrad():
    """26 tables of 1e6..1e7 rows, dim 64, batch 16384, bag length U[1,100] (about 21 M indices), SUM, Adagrad."""
    from recsdk_b200.synthetic import multi_hot_batch
    from recsdk_b200.tbe import EmbOptimType, PoolingMode

    T, D, B = 26, 64, 16384
    rows = _tables(7, T, 1e6, 1e7)
    gen = torch.Generator(device=DEV)
    gen.manual_seed(7)
    m = _module(rows, D, EmbOptimType.EXACT_ADAGRAD, PoolingMode.SUM, acc0=0.1)
    idx, offs = multi_hot_batch(gen, rows, B, 100, 1.2, DEV)
    assert idx.numel() > 15_000_000
    w0 = m.weights_dev.data.clone()
    acc0 = m.momentum1_dev.clone()
    out = torch.empty((B, T * D), device=DEV)
    m.forward_into(idx, offs, out)
    m.raise_if_error()
    tabs = m.split_embedding_weights()
    per = _per_table(idx, offs, T, B)
    for t in range(T):
        ref = torch.nn.functional.embedding_bag(per[t][0], tabs[t], per[t][1], mode="sum")
        torch.testing.assert_close(out[:, t * D:(t + 1) * D], ref, rtol=1e-6, atol=1e-6)
    grad = torch.randn((B, T * D), generator=gen, device=DEV)
    m.backward_from(grad, idx, offs)
    m.raise_if_error()
    w1 = m.weights_dev.data.clone()
    acc1 = m.momentum1_dev.clone()
    # independent computation: dense per-table gradient by index_add_, then the Adagrad formulas on touched rows
    off = 0
    for t in range(T):
        n = rows[t] * D
        lens = torch.diff(torch.cat([per[t][1], per[t][1].new_tensor([per[t][0].numel()])]))
        sample = torch.repeat_interleave(torch.arange(B, device=DEV), lens)
        g = torch.zeros((rows[t], D), device=DEV)
        g.index_add_(0, per[t][0], grad[:, t * D:(t + 1) * D][sample])
        touched = torch.zeros(rows[t], dtype=torch.bool, device=DEV)
        touched[per[t][0]] = True
        a_ref = acc0[off:off + n].view(rows[t], D) + g * g
        w_ref = w0[off:off + n].view(rows[t], D) - 0.01 * g / (a_ref.sqrt() + 1e-8)
        a_got, w_got = acc1[off:off + n].view(rows[t], D), w1[off:off + n].view(rows[t], D)
        scale = float(a_ref[touched].abs().max())
        assert float((a_got[touched] - a_ref[touched]).abs().max()) <= 2e-4 * max(scale, 1.0)
        assert float((w_got[touched] - w_ref[touched]).abs().max()) <= 2e-4
        # rows without an index this step are bit-identical
        assert torch.equal(w_got[~touched], w0[off:off + n].view(rows[t], D)[~touched])
        assert torch.equal(a_got[~touched], acc0[off:off + n].view(rows[t], D)[~touched])
        del g, a_ref, w_ref
        off += n
    # run-to-run bit identity: the same step from the same state gives the same bits
    m.weights_dev.data.copy_(w0)
    m.momentum1_dev.copy_(acc0)
    m.backward_from(grad, idx, offs)
    assert torch.equal(m.weights_dev.data, w1) and torch.equal(m.momentum1_dev, acc1)


def test_one_hot_config_full_size_adam_properties():
    """The benchmark's own workload (26 tables, dim 128, batch 65536 one-hot Zipf(1.1), Adam), rows capped at 2 M
    per table so that the dense torch reference fits beside it."""
    from recsdk_b200.synthetic import one_hot_batch
    from recsdk_b200.tbe import EmbOptimType, PoolingMode

    T, D, B = 26, 128, 65536
    rows = [min(r, 2_000_000) for r in _tables(2025, T, 1e3, 4e7)]
    gen = torch.Generator(device=DEV)
    gen.manual_seed(2025)
    m = _module(rows, D, EmbOptimType.ADAM, PoolingMode.SUM, lr=1e-3)
    idx, offs = one_hot_batch(gen, rows, B, 1.1, DEV)
    out = torch.empty((B, T * D), device=DEV)
    m.forward_into(idx, offs, out)
    tabs = m.split_embedding_weights()
    for t in range(T):
        # one id per bag: the pooled row is 0.0f + row, i.e. the row itself
        assert torch.equal(out[:, t * D:(t + 1) * D], tabs[t][idx[t * B:(t + 1) * B]])
    w0 = m.weights_dev.data.clone()
    grad = torch.randn((B, T * D), generator=gen, device=DEV)
    m.backward_from(grad, idx, offs)
    m.raise_if_error()
    w1, m1, m2 = m.weights_dev.data, m.momentum1_dev, m.momentum2_dev
    step = 1e-3 * float(np.sqrt(1 - 0.999) / (1 - 0.9))
    off = 0
    for t in range(T):
        n = rows[t] * D
        ids = idx[t * B:(t + 1) * B]
        g = torch.zeros((rows[t], D), device=DEV)
        g.index_add_(0, ids, grad[:, t * D:(t + 1) * D])
        touched = torch.zeros(rows[t], dtype=torch.bool, device=DEV)
        touched[ids] = True
        m1_ref = 0.1 * g
        m2_ref = 0.001 * g * g
        w_ref = w0[off:off + n].view(rows[t], D) - step * m1_ref / (m2_ref.sqrt() + 1e-8)
        tol = 2e-4 * max(float(g.abs().max()), 1.0)
        assert float((m1[off:off + n].view(rows[t], D)[touched] - m1_ref[touched]).abs().max()) <= tol
        assert float((m2[off:off + n].view(rows[t], D)[touched] - m2_ref[touched]).abs().max()) <= tol * tol + 1e-6
        # m1 / (sqrt(m2) + eps) is ill-conditioned where the summed gradient is ~0: compare w elsewhere
        firm = touched.view(-1, 1) & (g.abs() > 1e-3)
        assert float((w1[off:off + n].view(rows[t], D)[firm] - w_ref[firm]).abs().max()) <= 1e-5
        assert torch.equal(w1[off:off + n].view(rows[t], D)[~touched], w0[off:off + n].view(rows[t], D)[~touched])
        assert not bool(m1[off:off + n].view(rows[t], D)[~touched].any())
        del g, m1_ref, m2_ref, w_ref
        off += n
    U = m.last_num_unique()
    assert U == int(sum(torch.unique(idx[t * B:(t + 1) * B]).numel() for t in range(T)))


@pytest.mark.parametrize("eps", [1e-8, 0.0])
def test_config1_exact_size_bit_exact(eps):
    """The single-table config at its exact size -- 1,000,000 rows x 16, batch 4096 one-hot ids ~ Zipf(1.05) through a
    seeded permutation, N(0,1) upstream gradient, sparse Adagrad lr 0.01 with the accumulator starting at 0.1 -- in the
    torch flavour (eps 1e-8) and the TF flavour (eps 0: acc += g^2; w -= lr * g / sqrt(acc)), two steps, every bit of
    output, table and accumulator against the CPU oracle."""
    from oracle import port
    from recsdk_b200.tbe import EmbOptimType, HybridSplitTableBatchedEmbeddingBagsCodegen, PoolingMode
    from tests.golden.driver import zipf_ids

    rows, D, B = 1_000_000, 16, 4096
    rng = np.random.default_rng(1234)
    w = rng.uniform(-0.05, 0.05, rows * D).astype(np.float32)
    perm = rng.permutation(rows)
    m = HybridSplitTableBatchedEmbeddingBagsCodegen([(rows, D)], optimizer=EmbOptimType.EXACT_ADAGRAD,
                                                    pooling_mode=PoolingMode.SUM, device="cuda", learning_rate=0.01,
                                                    eps=eps, initial_accumulator_value=0.1)
    m.weights_dev.data.copy_(torch.from_numpy(w))
    acc = np.full_like(w, 0.1)
    wo, do, hs = np.zeros(1, np.int64), np.array([0, D], np.int32), np.array([0, rows], np.int64)
    offs = np.arange(B + 1, dtype=np.int64)
    for it in (1, 2):
        ids = perm[zipf_ids(rng, B, rows, 1.05)].astype(np.int64)
        grad = rng.standard_normal((B, D)).astype(np.float32)
        exp = port.tbe_forward(w, wo, do, ids, offs, 1, B, D, D, 0)
        out = m(torch.from_numpy(ids).cuda(), torch.from_numpy(offs).cuda())
        np.testing.assert_array_equal(out.detach().cpu().numpy(), exp)
        out.backward(torch.from_numpy(grad).cuda())
        port.tbe_backward(grad, w, acc, None, wo, do, hs, ids, offs, 1, B, D, D, 0, 1, 0.01, eps, reduce_chunk=64)
    np.testing.assert_array_equal(m.weights_dev.data.cpu().numpy(), w)
    np.testing.assert_array_equal(m.momentum1_dev.cpu().numpy(), acc)
