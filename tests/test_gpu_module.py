"""The module mirror of HybridSplitTableBatchedEmbeddingBagsCodegen: registered torch ops (fbgemm:: schemas) vs the
Python autograd Function vs the CPU oracle, swap helpers, and the recsdk:: IdsMapper torch class."""
import os

import numpy as np
import pytest
import torch

from oracle import port
from tests.golden.driver import zipf_ids

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _module(opt, mode, use_torch_ops, specs, seed=3, **kw):
    from recsdk_b200.tbe import EmbOptimType, HybridSplitTableBatchedEmbeddingBagsCodegen, PoolingMode

    o = {1: EmbOptimType.EXACT_ADAGRAD, 2: EmbOptimType.ADAM, 3: EmbOptimType.EXACT_SGD}[opt]
    return HybridSplitTableBatchedEmbeddingBagsCodegen(specs, optimizer=o, pooling_mode=PoolingMode(mode),
                                                       learning_rate=0.05, eps=1e-8, beta1=0.9, beta2=0.999, device=DEV,
                                                       weights_init=(-0.05, 0.05), seed=seed,
                                                       initial_accumulator_value=0.1 if opt == 1 else 0.0,
                                                       use_torch_ops=use_torch_ops, **kw)


@pytest.mark.parametrize("opt", [1, 2, 3])
@pytest.mark.parametrize("mode", [0, 1])
def test_registered_ops_match_python_function_and_oracle(opt, mode):
    from recsdk_b200 import torch_ops

    if not torch_ops.available():
        pytest.skip("torch op library not built")
    specs = [(300, 16), (500, 32), (200, 16)]
    rng = np.random.default_rng(opt * 10 + mode)
    B = 40
    a = _module(opt, mode, True, specs)
    b = _module(opt, mode, False, specs)
    assert a.use_torch_ops and not b.use_torch_ops
    assert torch.equal(a.weights_dev, b.weights_dev)
    w = a.weights_dev.detach().cpu().numpy().copy()
    m1 = np.full_like(w, 0.1 if opt == 1 else 0.0)
    m2 = np.zeros_like(w)
    T = len(specs)
    wo, do, hs = (x.cpu().numpy() for x in (a.weights_offsets, a.D_offsets, a.hash_size_cumsum))
    for step in range(3):
        lens = rng.integers(0, 5, T * B)
        offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        idx = np.concatenate([zipf_ids(rng, int(lens[t * B:(t + 1) * B].sum()), specs[t][0], 1.1) for t in range(T)])
        ti, to = torch.as_tensor(idx, device=DEV), torch.as_tensor(offs, device=DEV)
        oa, ob = a(ti, to), b(ti, to)
        exp = port.tbe_forward(w, wo, do, idx, offs, T, B, a.total_D, a.max_D, mode)
        np.testing.assert_array_equal(oa.detach().cpu().numpy(), exp)
        assert torch.equal(oa, ob)
        g = torch.as_tensor(rng.standard_normal(exp.shape).astype(np.float32), device=DEV)
        oa.backward(g)
        ob.backward(g)
        port.tbe_backward(g.cpu().numpy(), w, m1, m2, wo, do, hs, idx, offs, T, B, a.total_D, a.max_D, mode, opt, 0.05,
                          1e-8, 0.9, 0.999, step + 1, reduce_chunk=64)
    for mod in (a, b):
        np.testing.assert_array_equal(mod.weights_dev.detach().cpu().numpy(), w)
        if opt != 3:
            np.testing.assert_array_equal(mod.momentum1_dev.cpu().numpy(), m1)
        if opt == 2:
            np.testing.assert_array_equal(mod.momentum2_dev.cpu().numpy(), m2)
    assert int(a.iter.item()) == 3


def test_raw_registered_ops_and_errors():
    from recsdk_b200 import torch_ops

    if not torch_ops.available():
        pytest.skip("torch op library not built")
    torch_ops.load()
    w = torch.arange(8, dtype=torch.float32, device=DEV)
    e = torch.empty(0, device=DEV)
    ei = torch.empty(0, dtype=torch.int64, device=DEV)
    wo = torch.tensor([0], device=DEV)
    do = torch.tensor([0, 2], dtype=torch.int32, device=DEV)
    idx = torch.tensor([0, 1, 2, 3, 1], device=DEV)
    offs = torch.tensor([0, 2, 4, 5], device=DEV)
    pl = torch.zeros(1, dtype=torch.int32, device=DEV)
    for ns in (torch.ops.fbgemm, torch.ops.recsdk):
        # the schema's `Tensor x = None` defaults cannot be omitted from Python: pass empty tensors, as the C++ callers do
        out = ns.split_embedding_codegen_forward_unweighted_cuda(w, e, e, pl, wo, do, 2, 2, idx, offs, 0, e, e, 0, False, ei, ei)
        np.testing.assert_array_equal(out.cpu().numpy(), [[2, 4], [10, 12], [2, 3]])
    with pytest.raises(RuntimeError, match="incorrect for feature count"):
        torch.ops.fbgemm.split_embedding_codegen_forward_unweighted_cuda(
            w, e, e, torch.zeros(2, dtype=torch.int32, device=DEV), torch.tensor([0, 4], device=DEV),
            torch.tensor([0, 2, 4], dtype=torch.int32, device=DEV), 4, 2, idx, offs, 0, e, e, 0, False, ei, ei)
    # raw backward op (SGD, lr 1, grad 1): every touched row moves by its occurrence count
    g = torch.ones(3, 2, device=DEV)
    hs = torch.tensor([0, 4], device=DEV)
    r = torch.ops.fbgemm.split_embedding_backward_codegen_sgd_unweighted_exact_cuda(
        g, w, e, e, pl, wo, do, 2, hs, 3, idx, offs, 0, e, 32, 32, False, 0, 0, False, False, ei, ei, ei, ei, ei, 1.0)
    np.testing.assert_array_equal(w.cpu().numpy().reshape(4, 2), [[-1, 0], [0, 1], [3, 4], [5, 6]])


def test_swap_helpers():
    m = _module(2, 0, False, [(1000, 32), (500, 32)])
    rng = np.random.default_rng(0)
    slots = torch.as_tensor(rng.permutation(1500)[:200].astype(np.int64), device=DEV)
    rows = m.gather_embs(slots)
    assert torch.equal(rows.view(-1, 32), m.weights_dev.view(-1, 32)[slots])
    new = torch.randn(200, 32, device=DEV)
    m.scatter_update_embs(slots, new)
    assert torch.equal(m.weights_dev.view(-1, 32)[slots], new)
    m.scatter_update_momentum(slots, [new, new * 2])
    g1, g2 = m.gather_momentum(slots)
    assert torch.equal(g1.view(-1, 32), new) and torch.equal(g2.view(-1, 32), new * 2)
    mixed = _module(3, 0, False, [(10, 8), (10, 16)])
    with pytest.raises(ValueError, match="Mixed dimensions"):
        mixed.gather_embs(slots[:2])


@pytest.mark.parametrize("ns", ["recsdk", "hybrid"])
def test_ids_mapper_torch_class_matches_reference_golden(golden_dir, ns):
    """`hybrid` is the reference's own registration name (hybrid_torchrec/src/bind_torch_lib.cpp:9-19)."""
    from recsdk_b200 import torch_ops

    if not torch_ops.available():
        pytest.skip("torch op library not built")
    torch_ops.load()
    IdsMapper = getattr(torch.classes, ns).IdsMapper
    g = np.load(os.path.join(golden_dir, "ids_mapper.npz"))
    T = 3
    mappers = [IdsMapper(4096, True) for _ in range(T)]
    for s in range(3):
        ids = torch.as_tensor(g[f"s{s}_ids"], device=DEV)
        offset = torch.as_tensor(g[f"s{s}_offset"])
        n = ids.numel()
        hi, uq, uid, inv = (torch.full((max(n, 1),), -7, dtype=torch.int64, device=DEV) for _ in range(4))
        uoff = torch.zeros(T + 1, dtype=torch.int64, device=DEV)
        if s == 2:
            IdsMapper.parallel_ids2indices_unique_out(mappers, ids, hi, offset, uq, uid, inv, uoff)
        else:
            for t in range(T):
                mappers[t].ids2indices_unique_out(ids, hi, offset, uq, uid, inv, uoff, t)
        U = int(uoff[-1].item())
        np.testing.assert_array_equal(uoff.cpu().numpy(), g[f"s{s}_unique_offset"])
        np.testing.assert_array_equal(hi.cpu().numpy()[:n], g[f"s{s}_hash_indices"])
        np.testing.assert_array_equal(uq.cpu().numpy()[:U], g[f"s{s}_unique"])
        np.testing.assert_array_equal(uid.cpu().numpy()[:U], g[f"s{s}_unique_ids"])
        np.testing.assert_array_equal(inv.cpu().numpy()[:n], g[f"s{s}_unique_inverse"])
    m = IdsMapper(100000, True)
    for s in range(2):
        hi, uq, inv = m.ids2indices_unique(torch.as_tensor(g[f"u{s}_ids"], device=DEV))
        np.testing.assert_array_equal(hi.cpu().numpy(), g[f"u{s}_hash_indices"])
        np.testing.assert_array_equal(uq.cpu().numpy(), g[f"u{s}_unique"])
    with pytest.raises(RuntimeError, match="Invalid key value"):
        IdsMapper(8, True).ids2indices_unique(torch.tensor([3, -2], device=DEV))


@pytest.mark.parametrize("op", ["recsdk.block_bucketize_sparse_features", "hybrid.block_bucketize_sparse_features_cpu"])
def test_bucketize_torch_op_matches_reference_golden(golden_dir, op):
    from recsdk_b200 import torch_ops

    if not torch_ops.available():
        pytest.skip("torch op library not built")
    torch_ops.load()
    g = np.load(os.path.join(golden_dir, "bucketize.npz"))
    for c in range(int(g["n_cases"][0])):
        W, F, B, do_unique, ret_count = (int(x) for x in g[f"c{c}_meta"])
        ns, name = op.split(".")
        res = getattr(getattr(torch.ops, ns), name)(
            torch.as_tensor(g[f"c{c}_lengths"], device=DEV), torch.as_tensor(g[f"c{c}_indices"], device=DEV), False, True,
            torch.ones(F, dtype=torch.int64), W, None, None, None, 0, None, False, False, bool(do_unique), bool(ret_count))
        np.testing.assert_array_equal(res[0].cpu().numpy(), g[f"c{c}_new_lengths"])
        np.testing.assert_array_equal(res[1].cpu().numpy(), g[f"c{c}_new_indices"])
        np.testing.assert_array_equal(res[4].cpu().numpy(), g[f"c{c}_unbucketize_permute"])
        np.testing.assert_array_equal(res[6].cpu().numpy(), g[f"c{c}_ids_counts"])


@pytest.mark.parametrize("mode", [0, 1])
def test_module_plan_ahead_matches_plain_module(mode):
    """plan_ahead=True (the backward's index work enqueued on a side stream by every forward) through autograd and
    through forward_into / backward_from: same weights, bit for bit, as the module without it."""
    from recsdk_b200.tbe import EmbOptimType, HybridSplitTableBatchedEmbeddingBagsCodegen, PoolingMode

    specs = [(500, 128), (40, 128), (300, 64)]
    mods = [HybridSplitTableBatchedEmbeddingBagsCodegen(specs, optimizer=EmbOptimType.ADAM, pooling_mode=PoolingMode(mode),
                                                        learning_rate=0.05, device=DEV, weights_init=(-0.1, 0.1), seed=4,
                                                        plan_ahead=pa) for pa in (False, True)]
    rng = np.random.default_rng(mode)
    B = 64
    for step in range(4):
        lens = rng.integers(0, 4, 3 * B)
        offs = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)).to(DEV)
        idx = torch.from_numpy(np.concatenate([rng.integers(0, specs[i // B][0] if i % 5 else 7, lens[i])
                                               for i in range(3 * B)]).astype(np.int64)).to(DEV)
        g = torch.randn(B, 128 + 128 + 64, device=DEV)
        for m in mods:
            if step % 2 == 0:
                out = m(idx, offs)
                out.backward(g)
            else:
                out = torch.empty(B, 320, device=DEV)
                m.forward_into(idx, offs, out)
                m.backward_from(g, idx, offs)
    assert torch.equal(mods[0].weights_dev.data, mods[1].weights_dev.data)
    assert torch.equal(mods[0].momentum1_dev, mods[1].momentum1_dev)
    assert torch.equal(mods[0].momentum2_dev, mods[1].momentum2_dev)


@pytest.mark.parametrize("plan_ahead", [False, True])
def test_module_step_as_cuda_graph_same_bits(plan_ahead):
    """capture_step: forward_into + backward_from replayed as one CUDA graph, the static index buffers refilled before
    every replay -- the same outputs, weights and accumulator, bit for bit, as the module stepped call by call."""
    from recsdk_b200.tbe import EmbOptimType, HybridSplitTableBatchedEmbeddingBagsCodegen, PoolingMode

    specs = [(1000, 16), (50, 16)]
    B = 128
    mods = [HybridSplitTableBatchedEmbeddingBagsCodegen(specs, optimizer=EmbOptimType.EXACT_ADAGRAD,
                                                        pooling_mode=PoolingMode.SUM, learning_rate=0.05, device=DEV,
                                                        initial_accumulator_value=0.1, weights_init=(-0.1, 0.1), seed=9,
                                                        plan_ahead=plan_ahead) for _ in range(2)]
    rng = np.random.default_rng(12)
    offs = torch.arange(2 * B + 1, dtype=torch.int64, device=DEV)  # one id per bag

    def batch():
        idx = np.concatenate([rng.integers(0, 1000, B) % np.where(rng.random(B) < 0.3, 5, 1000), rng.integers(0, 50, B)])
        return torch.from_numpy(idx.astype(np.int64)).to(DEV), torch.randn(B, 32, device=DEV)

    outs = [torch.empty(B, 32, device=DEV) for _ in range(2)]
    idx, g = batch()
    for m, o in zip(mods, outs):  # one ordinary step first
        m.forward_into(idx, offs, o)
        m.backward_from(g, idx, offs)
    s_idx, s_g = idx.clone(), g.clone()
    graph = mods[1].capture_step(s_idx, offs, outs[1], s_g)
    for _ in range(5):
        idx, g = batch()
        mods[0].forward_into(idx, offs, outs[0])
        mods[0].backward_from(g, idx, offs)
        s_idx.copy_(idx)
        s_g.copy_(g)
        graph.replay()
        assert torch.equal(outs[0], outs[1])
    assert torch.equal(mods[0].weights_dev.data, mods[1].weights_dev.data)
    assert torch.equal(mods[0].momentum1_dev, mods[1].momentum1_dev)
    adam = HybridSplitTableBatchedEmbeddingBagsCodegen(specs, optimizer=EmbOptimType.ADAM, device=DEV)
    with pytest.raises(RuntimeError, match="Adam"):
        adam.capture_step(s_idx, offs, outs[0], s_g)


def test_registered_ops_plan_ahead_same_bits():
    """recsdk::set_plan_ahead(True): the registered lookup operators enqueue their backward's index work on a side
    stream during the forward.  Same weights, bit for bit, as with the switch off."""
    from recsdk_b200 import torch_ops
    from recsdk_b200.tbe import EmbOptimType, HybridSplitTableBatchedEmbeddingBagsCodegen, PoolingMode

    if not torch_ops.available():
        pytest.skip("torch op library not built")
    torch_ops.load()
    specs = [(500, 128), (40, 128), (300, 64)]
    rng = np.random.default_rng(12)
    B = 64
    steps = []
    for _ in range(4):
        lens = rng.integers(0, 4, 3 * B)
        offs = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)).to(DEV)
        idx = torch.from_numpy(np.concatenate([rng.integers(0, specs[i // B][0] if i % 5 else 7, lens[i])
                                               for i in range(3 * B)]).astype(np.int64)).to(DEV)
        steps.append((idx, offs, torch.randn(B, 320, device=DEV)))
    results = []
    try:
        for on in (False, True):
            torch.ops.recsdk.set_plan_ahead(on)
            assert torch.ops.recsdk.get_plan_ahead() == on
            m = HybridSplitTableBatchedEmbeddingBagsCodegen(specs, optimizer=EmbOptimType.ADAM, pooling_mode=PoolingMode.SUM,
                                                            learning_rate=0.05, device=DEV, weights_init=(-0.1, 0.1), seed=4,
                                                            use_torch_ops=True)
            for idx, offs, g in steps:
                m(idx, offs).backward(g)
            torch.cuda.synchronize()
            results.append((m.weights_dev.data.clone(), m.momentum1_dev.clone(), m.momentum2_dev.clone()))
    finally:
        torch.ops.recsdk.set_plan_ahead(False)
    for a, b in zip(*results):
        assert torch.equal(a, b)


def test_tf_flavour_torch_operators_match_oracle():
    """torch.ops.recsdk.{EmbeddingLookupByAddress, EmbeddingUpdateByAddress, LazyAdam, Sgd}: the reference's TF operator
    signatures (cust_op/framework/tf_plugin/src/*.cpp) as torch operators, bit for bit against the oracle."""
    from oracle import port
    from recsdk_b200 import torch_ops

    if not torch_ops.available():
        pytest.skip("torch op library not built")
    torch_ops.load()
    rng = np.random.default_rng(21)
    rows, dim, n = 5000, 16, 700
    table_np = rng.standard_normal((rows, dim)).astype(np.float32)
    table = torch.from_numpy(table_np).cuda()
    slots = rng.permutation(rows)[:n]
    addr = table.data_ptr() + slots.astype(np.int64) * dim * 4
    addr[::50] = 0
    out = torch.ops.recsdk.EmbeddingLookupByAddress(torch.from_numpy(addr).cuda(), dim, 0)
    exp = table_np[slots].copy()
    exp[::50] = 0
    np.testing.assert_array_equal(out.cpu().numpy(), exp)
    upd = rng.standard_normal((n, dim)).astype(np.float32)
    torch.ops.recsdk.EmbeddingUpdateByAddress(torch.from_numpy(addr).cuda(), torch.from_numpy(upd).cuda(), 1)
    e2 = table_np.copy()
    live = addr != 0
    e2[slots[live]] = upd[live]
    np.testing.assert_array_equal(table.cpu().numpy(), e2)

    m, v, var = (rng.uniform(1, 2, (rows, dim)).astype(np.float32) for _ in range(3))
    g = rng.uniform(1, 2, (n, dim)).astype(np.float32)
    idx = slots.astype(np.int32)
    idx[3] = -1
    dm, dv, dvar = (torch.from_numpy(a.copy()).cuda() for a in (m, v, var))
    om, ov, ovar = torch.ops.recsdk.LazyAdam(torch.from_numpy(g).cuda(), torch.from_numpy(idx).cuda(), dm, dv, dvar,
                                             torch.tensor(1e-3), 0.9, 0.999, 1e-7)
    port.lazy_adam(g, idx, m, v, var, 1e-3, 0.9, 0.999, 1e-7)
    assert om.data_ptr() == dm.data_ptr() and ovar.data_ptr() == dvar.data_ptr()  # state updated in place
    for a, b in ((dm, m), (dv, v), (dvar, var)):
        np.testing.assert_array_equal(a.cpu().numpy(), b)

    var2 = rng.standard_normal((rows, dim)).astype(np.float32)
    dvar2 = torch.from_numpy(var2.copy()).cuda()
    idx64 = slots.astype(np.int64)
    torch.ops.recsdk.Sgd(torch.from_numpy(g).cuda(), torch.from_numpy(idx64.astype(np.int32)).cuda(), dvar2,
                         torch.tensor(0.1), 0.01)
    port.sgd(g, idx64, var2, 0.1, 0.01)
    np.testing.assert_array_equal(dvar2.cpu().numpy(), var2)
