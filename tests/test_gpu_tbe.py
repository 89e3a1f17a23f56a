"""Parity of the CUDA forward / fused backward (through the C ABI) with the CPU oracle.
Integer outputs and gathered rows must be bit-exact; float results are bit-exact too because both
sides fix the same reduction order (reduce_chunk 0: sequential; 64: chunked) and operand order."""
import os

import numpy as np
import pytest
import torch

from oracle import port
from tests.golden.driver import zipf_ids

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _t(a, dtype=None):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=dtype).to(DEV)


def make_case(rng, rows, dims, B, max_len, alpha=1.05, feature_table_map=None, empty_frac=0.1, one_hot=False):
    """Returns dict with layout arrays + random indices/offsets (feature-major)."""
    n_tables = len(rows)
    ftm = list(range(n_tables)) if feature_table_map is None else feature_table_map
    T = len(ftm)
    table_wo = np.concatenate([[0], np.cumsum([r * d for r, d in zip(rows, dims)])]).astype(np.int64)
    table_hs = np.concatenate([[0], np.cumsum(rows)]).astype(np.int64)
    wo = np.array([table_wo[t] for t in ftm], np.int64)
    fd = [dims[t] for t in ftm]
    do = np.concatenate([[0], np.cumsum(fd)]).astype(np.int32)
    # hash_size_cumsum per feature (features of one table share the entry), plus the total at the end
    hs = np.array([table_hs[t] for t in ftm] + [table_hs[-1]], np.int64)
    idx_all, lens_all = [], []
    for f in range(T):
        if one_hot:
            lens = np.ones(B, np.int64)
        else:
            lens = rng.integers(0 if empty_frac > 0 else 1, max_len + 1, size=B)
            lens[rng.random(B) < empty_frac] = 0
        idx_all.append(zipf_ids(rng, int(lens.sum()), rows[ftm[f]], alpha))
        lens_all.append(lens)
    indices = np.concatenate(idx_all).astype(np.int64)
    offsets = np.concatenate([[0], np.cumsum(np.concatenate(lens_all))]).astype(np.int64)
    w = rng.uniform(-0.05, 0.05, int(table_wo[-1])).astype(np.float32)
    return dict(T=T, B=B, wo=wo, do=do, hs=hs, indices=indices, offsets=offsets, w=w, total_D=int(do[-1]),
                max_D=max(fd), dims=fd, rows=rows, ftm=ftm)


FWD_CASES = [
    dict(rows=[50], dims=[8], B=7, max_len=3),
    dict(rows=[1000], dims=[16], B=64, max_len=1, one_hot=True),
    dict(rows=[200, 300, 120], dims=[8, 16, 8], B=33, max_len=6),
    dict(rows=[400, 500], dims=[32, 32], B=50, max_len=12),
    dict(rows=[4000, 8000], dims=[128, 128], B=100, max_len=20),
    dict(rows=[300], dims=[64], B=40, max_len=100, empty_frac=0.0),
    dict(rows=[100], dims=[256], B=9, max_len=5),
    dict(rows=[64], dims=[1024], B=5, max_len=4),
    dict(rows=[77], dims=[1536], B=4, max_len=3),
    dict(rows=[1], dims=[8], B=3, max_len=2),
    dict(rows=[90, 60], dims=[6, 10], B=11, max_len=4),  # dims not multiples of 4: scalar path
    dict(rows=[100, 200], dims=[16, 16], B=20, max_len=5, feature_table_map=[0, 0, 1]),
]


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("case", range(len(FWD_CASES)))
def test_forward_bit_exact(case, mode):
    rng = np.random.default_rng(1000 + case)
    c = make_case(rng, **FWD_CASES[case])
    from recsdk_b200 import ops

    exp = port.tbe_forward(c["w"], c["wo"], c["do"], c["indices"], c["offsets"], c["T"], c["B"], c["total_D"],
                           c["max_D"], mode)
    st = ops.new_status(DEV)
    out = ops.tbe_forward(_t(c["w"]), _t(c["wo"]), _t(c["do"]), _t(c["indices"]), _t(c["offsets"]), c["total_D"],
                          c["max_D"], mode, status=st)
    ops.raise_on_status(st)
    np.testing.assert_array_equal(out.cpu().numpy(), exp)


def test_forward_hand_examples():
    """hybrid_torchrec/test/dt/test_batched_embedding_kernel.py:42-46"""
    from recsdk_b200 import ops

    w = torch.arange(8, dtype=torch.float32, device=DEV)
    out = ops.tbe_forward(w, _t([0]), _t([0, 2], torch.int32), _t([0, 1, 2, 3, 1]), _t([0, 2, 4, 5]), 2, 2, 0)
    np.testing.assert_array_equal(out.cpu().numpy(), [[2, 4], [10, 12], [2, 3]])


def test_forward_out_of_range_sets_status():
    from recsdk_b200 import ops

    w = torch.zeros(8, dtype=torch.float32, device=DEV)
    st = ops.new_status(DEV)
    ops.tbe_forward(w, _t([0]), _t([0, 2], torch.int32), _t([0, 9]), _t([0, 1, 2]), 2, 2, 0, status=st)
    with pytest.raises(RuntimeError, match="out of range"):
        ops.raise_on_status(st)


def test_forward_bad_offsets_raises():
    from recsdk_b200 import ops

    w = torch.zeros(8, dtype=torch.float32, device=DEV)
    with pytest.raises(RuntimeError, match="incorrect for feature count"):
        ops.tbe_forward(w, _t([0, 4]), _t([0, 2, 4], torch.int32), _t([0]), _t([0, 1, 1, 1]), 4, 2, 0)


def _unique_inputs(c, first_occurrence):
    """Per-table unique ids / inverse / offsets expanded per feature like do_unique_hash_out
    (hybrid_torchrec/distributed/sharding/post_input_dist.py:255-262)."""
    T, B = c["T"], c["B"]
    ftm = c["ftm"]
    n_tables = len(c["rows"])
    uids, uoff_single = [], [0]
    inv = np.empty(c["indices"].size, np.int64)
    for tb in range(n_tables):
        feats = [f for f in range(T) if ftm[f] == tb]
        segs = [(c["offsets"][f * B], c["offsets"][(f + 1) * B]) for f in feats]
        ids = np.concatenate([c["indices"][s:e] for s, e in segs]) if segs else np.empty(0, np.int64)
        if first_occurrence:
            _, first = np.unique(ids, return_index=True)
            u = ids[np.sort(first)]
            lut = {int(v): k for k, v in enumerate(u)}
            iv = np.array([lut[int(v)] for v in ids], np.int64)
        else:
            u, iv = port.unique_sorted(ids)
        k = 0
        for s, e in segs:
            inv[s:e] = iv[k:k + (e - s)]
            k += e - s
        uids.append(u)
        uoff_single.append(uoff_single[-1] + u.size)
    uoff = []
    for tb in range(n_tables):
        nf = sum(1 for f in range(T) if ftm[f] == tb)
        uoff.extend([uoff_single[tb]] * nf)
    uoff.append(uoff_single[-1])
    return np.concatenate(uids).astype(np.int64), np.array(uoff, np.int64), inv


BWD_CASES = [
    dict(rows=[50], dims=[8], B=7, max_len=3),
    dict(rows=[1000], dims=[16], B=256, max_len=1, one_hot=True),
    dict(rows=[200, 300, 120], dims=[8, 16, 8], B=33, max_len=6),
    dict(rows=[40, 8000], dims=[128, 128], B=300, max_len=3, alpha=1.3),  # hot rows: runs > 64
    dict(rows=[30], dims=[64], B=50, max_len=40, empty_frac=0.0),        # very hot rows
    dict(rows=[64], dims=[1024], B=5, max_len=4),
    dict(rows=[90, 60], dims=[6, 10], B=11, max_len=4),
    dict(rows=[100, 200], dims=[16, 16], B=20, max_len=5, feature_table_map=[0, 0, 1]),
    dict(rows=[20, 100], dims=[256, 256], B=70, max_len=4),
    # features 0 and 2 share table 0 (dim 8) but feature 2's gradient columns start at 14: one run holds gradient
    # rows of both, so the whole call must take the scalar path
    dict(rows=[60, 40, 30], dims=[8, 6, 2], B=25, max_len=4, feature_table_map=[0, 1, 0, 2]),
]


@pytest.mark.parametrize("chunk", [0, 64])
@pytest.mark.parametrize("unique", ["none", "sorted", "first"])
@pytest.mark.parametrize("opt", [1, 2, 3])
@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("case", range(len(BWD_CASES)))
def test_backward_bit_exact(case, mode, opt, unique, chunk):
    if mode == 2 and len(set(BWD_CASES[case]["dims"])) > 1:
        pytest.skip("NONE pooling needs equal dims (grad rows are max_D wide)")
    ftm = BWD_CASES[case].get("feature_table_map")
    if unique != "none" and ftm is not None and any(ftm[i] in ftm[:i] and ftm[i - 1] != ftm[i] for i in range(1, len(ftm))):
        pytest.skip("caller-side unique lists need the features of one table to be adjacent (monotonic unique_offsets)")
    rng = np.random.default_rng(2000 + case)
    c = make_case(rng, **BWD_CASES[case])
    from recsdk_b200 import ops

    N = c["indices"].size
    gshape = (N, c["max_D"]) if mode == 2 else (c["B"], c["total_D"])
    grad = rng.standard_normal(gshape).astype(np.float32)
    w = c["w"].copy()
    m1 = np.full_like(w, 0.1) if opt == 1 else rng.uniform(0, 0.01, w.size).astype(np.float32)
    m2 = rng.uniform(0, 0.01, w.size).astype(np.float32)
    kw = {}
    if unique != "none":
        uid, uoff, inv = _unique_inputs(c, unique == "first")
        kw = dict(unique_ids=uid, unique_offsets=uoff, unique_inverse=inv)
    hp = dict(lr=0.05, eps=1e-8, beta1=0.9, beta2=0.999)
    dw, dm1, dm2 = _t(w), _t(m1), _t(m2)
    ew, em1, em2 = w.copy(), m1.copy(), m2.copy()
    st = ops.new_status(DEV)
    bits = int(c["hs"][-1]).bit_length()
    for it in (1, 2):
        port.tbe_backward(grad, ew, em1, em2, c["wo"], c["do"], c["hs"], c["indices"], c["offsets"], c["T"], c["B"],
                          c["total_D"], c["max_D"], mode, opt, hp["lr"], hp["eps"], hp["beta1"], hp["beta2"], it,
                          reduce_chunk=chunk, **kw)
        ops.tbe_backward(_t(grad), dw, dm1, dm2, _t(c["wo"]), _t(c["do"]), _t(c["hs"]), _t(c["indices"]),
                         _t(c["offsets"]), c["total_D"], c["max_D"], mode, opt, hp["lr"], hp["eps"], hp["beta1"],
                         hp["beta2"], it, total_hash_size_bits=bits, reduce_chunk=chunk, status=st,
                         **{k: _t(v) for k, v in kw.items()})
    ops.raise_on_status(st)
    np.testing.assert_array_equal(dw.cpu().numpy(), ew)
    if opt != 3:
        np.testing.assert_array_equal(dm1.cpu().numpy(), em1)
    if opt == 2:
        np.testing.assert_array_equal(dm2.cpu().numpy(), em2)


@pytest.mark.parametrize("opt", [1, 2, 3])
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("case", [3, 5, 8])
def test_backward_staged_update_bit_exact(case, mode, opt):
    """RECSDK_BWD_STAGED_UPDATE (rows moved through shared memory by bulk asynchronous copies) gives the same bits
    as the default update; shapes of 128, 256 and 1024 floats per row, hot rows included."""
    rng = np.random.default_rng(2500 + case)
    c = make_case(rng, **BWD_CASES[case])
    from recsdk_b200 import ops

    grad = rng.standard_normal((c["B"], c["total_D"])).astype(np.float32)
    w = c["w"].copy()
    m1 = np.full_like(w, 0.1) if opt == 1 else rng.uniform(0, 0.01, w.size).astype(np.float32)
    m2 = rng.uniform(0, 0.01, w.size).astype(np.float32)
    dw, dm1, dm2 = _t(w), _t(m1), _t(m2)
    st = ops.new_status(DEV)
    bits = int(c["hs"][-1]).bit_length()
    for it in (1, 2, 3):
        port.tbe_backward(grad, w, m1, m2, c["wo"], c["do"], c["hs"], c["indices"], c["offsets"], c["T"], c["B"],
                          c["total_D"], c["max_D"], mode, opt, 0.05, 1e-8, 0.9, 0.999, it, reduce_chunk=64)
        ops.tbe_backward(_t(grad), dw, dm1, dm2, _t(c["wo"]), _t(c["do"]), _t(c["hs"]), _t(c["indices"]),
                         _t(c["offsets"]), c["total_D"], c["max_D"], mode, opt, 0.05, 1e-8, 0.9, 0.999, it,
                         total_hash_size_bits=bits, reduce_chunk=64, status=st, staged_update=True)
    ops.raise_on_status(st)
    np.testing.assert_array_equal(dw.cpu().numpy(), w)
    if opt != 3:
        np.testing.assert_array_equal(dm1.cpu().numpy(), m1)
    if opt == 2:
        np.testing.assert_array_equal(dm2.cpu().numpy(), m2)


@pytest.mark.parametrize("opt", [1, 2])
@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("case", [2, 3, 7, 8])
def test_backward_plan_then_apply_bit_exact(case, mode, opt):
    """RECSDK_BWD_PLAN_ONLY on a side stream (no gradient given), then RECSDK_BWD_APPLY_ONLY on the main stream
    after an event: same bits as the single call, i.e. as the oracle."""
    if mode == 2 and len(set(BWD_CASES[case]["dims"])) > 1:
        pytest.skip("NONE pooling needs equal dims")
    rng = np.random.default_rng(2600 + case)
    c = make_case(rng, **BWD_CASES[case])
    from recsdk_b200 import ops

    N = c["indices"].size
    gshape = (N, c["max_D"]) if mode == 2 else (c["B"], c["total_D"])
    grad = rng.standard_normal(gshape).astype(np.float32)
    w = c["w"].copy()
    m1 = np.full_like(w, 0.1) if opt == 1 else rng.uniform(0, 0.01, w.size).astype(np.float32)
    m2 = rng.uniform(0, 0.01, w.size).astype(np.float32)
    dw, dm1, dm2 = _t(w), _t(m1), _t(m2)
    st = ops.new_status(DEV)
    bits = int(c["hs"][-1]).bit_length()
    ws = torch.empty(ops.tbe_backward_workspace_bytes(N, c["max_D"]), dtype=torch.uint8, device=DEV)
    side, ev = torch.cuda.Stream(), torch.cuda.Event()
    d = dict(wo=_t(c["wo"]), do=_t(c["do"]), hs=_t(c["hs"]), idx=_t(c["indices"]), offs=_t(c["offsets"]), g=_t(grad))
    for it in (1, 2):
        port.tbe_backward(grad, w, m1, m2, c["wo"], c["do"], c["hs"], c["indices"], c["offsets"], c["T"], c["B"],
                          c["total_D"], c["max_D"], mode, opt, 0.05, 1e-8, 0.9, 0.999, it, reduce_chunk=64)
        args = (dw, dm1, dm2, d["wo"], d["do"], d["hs"], d["idx"], d["offs"], c["total_D"], c["max_D"], mode, opt, 0.05,
                1e-8, 0.9, 0.999, it)
        kw = dict(total_hash_size_bits=bits, reduce_chunk=64, status=st, workspace=ws)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ops.tbe_backward(None, *args, phase="plan", **kw)
            ev.record(side)
        torch.cuda.current_stream().wait_event(ev)
        ops.tbe_backward(d["g"], *args, phase="apply", **kw)
    ops.raise_on_status(st)
    np.testing.assert_array_equal(dw.cpu().numpy(), w)
    np.testing.assert_array_equal(dm1.cpu().numpy(), m1)
    if opt == 2:
        np.testing.assert_array_equal(dm2.cpu().numpy(), m2)
    with pytest.raises(RuntimeError, match="workspace"):
        ops.tbe_backward(None, *args, phase="plan", total_hash_size_bits=bits)


def test_backward_gradient_clipping_and_64bit_keys():
    rng = np.random.default_rng(7)
    c = make_case(rng, rows=[300, 200], dims=[16, 16], B=40, max_len=5)
    from recsdk_b200 import ops

    grad = (rng.standard_normal((c["B"], c["total_D"])) * 3).astype(np.float32)
    w, m1 = c["w"].copy(), np.full_like(c["w"], 0.1)
    dw, dm1 = _t(w), _t(m1)
    port.tbe_backward(grad, w, m1, None, c["wo"], c["do"], c["hs"], c["indices"], c["offsets"], c["T"], c["B"],
                      c["total_D"], c["max_D"], 0, 1, 0.01, 1e-8, gradient_clipping=True, max_gradient=0.5,
                      reduce_chunk=64)
    # total_hash_size_bits = 0 -> 64-bit sort keys
    ops.tbe_backward(_t(grad), dw, dm1, None, _t(c["wo"]), _t(c["do"]), _t(c["hs"]), _t(c["indices"]),
                     _t(c["offsets"]), c["total_D"], c["max_D"], 0, 1, 0.01, 1e-8, gradient_clipping=True,
                     max_gradient=0.5, total_hash_size_bits=0)
    np.testing.assert_array_equal(dw.cpu().numpy(), w)
    np.testing.assert_array_equal(dm1.cpu().numpy(), m1)


def test_tbe_vs_torch_golden(golden_dir):
    """The reference operator test's golden (nn.EmbeddingBag + torch.optim, 4 epochs, loss = sum(out^2)/2)
    at its gate: isclose(1e-4, 1e-4)."""
    from recsdk_b200 import ops

    g = np.load(os.path.join(golden_dir, "tbe_torch.npz"))
    specs = g["specs"]
    rows = [int(r) for r, _ in specs]
    dims = [int(d) for _, d in specs]
    wo = np.concatenate([[0], np.cumsum([r * d for r, d in zip(rows, dims)])])[:-1].astype(np.int64)
    do = np.concatenate([[0], np.cumsum(dims)]).astype(np.int32)
    hs = np.concatenate([[0], np.cumsum(rows)]).astype(np.int64)
    total_D, max_D = int(do[-1]), max(dims)
    for c in range(int(g["n_cases"][0])):
        mode, opt, B, epochs = (int(x) for x in g[f"c{c}_meta"])
        w = _t(g[f"c{c}_w0"].astype(np.float32))
        m1 = torch.full_like(w, 0.1 if opt == 1 else 0.0)
        m2 = torch.zeros_like(w)
        lr = {1: 0.05, 2: 0.01, 3: 0.05}[opt]
        for e in range(epochs):
            idx, offs = _t(g[f"c{c}_e{e}_indices"]), _t(g[f"c{c}_e{e}_offsets"])
            out = ops.tbe_forward(w, _t(wo), _t(do), idx, offs, total_D, max_D, mode)
            np.testing.assert_allclose(out.cpu().numpy(), g[f"c{c}_e{e}_out"], rtol=1e-4, atol=1e-4)
            ops.tbe_backward(out, w, m1, m2, _t(wo), _t(do), _t(hs), idx, offs, total_D, max_D, mode, opt, lr,
                             1e-8, 0.9, 0.999, e + 1, total_hash_size_bits=11)
        np.testing.assert_allclose(w.cpu().numpy(), g[f"c{c}_w_final"], rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("n,bits,vocab", [(1, 64, 10), (5000, 64, 2**62), (100000, 20, 2**20), (70000, 33, 2**33),
                                          (4096, 8, 200)])
def test_unique_sorted_bit_exact(n, bits, vocab):
    from recsdk_b200 import ops

    rng = np.random.default_rng(n)
    ids = rng.integers(0, vocab, size=n, dtype=np.int64)
    if n > 10:
        ids[: n // 2] = ids[n // 2: n // 2 * 2][: n // 2]  # force duplicates
    eu, einv = port.unique_sorted(ids)
    uq, inv, cnt = ops.unique_sorted(_t(ids), key_bits=bits)
    u = int(cnt.item())
    assert u == eu.size
    np.testing.assert_array_equal(uq[:u].cpu().numpy(), eu)
    np.testing.assert_array_equal(inv.cpu().numpy(), einv)


def test_unique_sorted_empty():
    from recsdk_b200 import ops

    uq, inv, cnt = ops.unique_sorted(torch.empty(0, dtype=torch.int64, device=DEV))
    assert int(cnt.item()) == 0 and inv.numel() == 0


def test_full_size_properties_config2_shape():
    """At the benchmark's shape (dim 128, one-hot, Adam) check size-independent properties:
    SGD with lr=1 on grad=1 subtracts the occurrence count of each row (a checksum of the
    segment-sum), and forward rows equal the table rows they index."""
    from recsdk_b200 import ops

    rng = np.random.default_rng(11)
    T, B, D = 4, 65536, 128
    rows = [1000, 50000, 300000, 2000000]
    wo = np.concatenate([[0], np.cumsum([r * D for r in rows])]).astype(np.int64)
    hs = np.concatenate([[0], np.cumsum(rows)]).astype(np.int64)
    do = (np.arange(T + 1) * D).astype(np.int32)
    idx = np.concatenate([zipf_ids(rng, B, r, 1.1) for r in rows]).astype(np.int64)
    offs = np.arange(T * B + 1, dtype=np.int64)
    w = torch.zeros(int(wo[-1]), dtype=torch.float32, device=DEV)
    w.uniform_(-0.01, 0.01)
    w0 = w.clone()
    out = ops.tbe_forward(w, _t(wo[:-1]), _t(do), _t(idx), _t(offs), T * D, D, 0)
    for t in range(T):
        sel = torch.as_tensor(idx[t * B:(t + 1) * B], device=DEV)
        exp = w0[wo[t]:wo[t + 1]].view(rows[t], D)[sel]
        assert torch.equal(out[:, t * D:(t + 1) * D], exp)
    grad = torch.ones((B, T * D), dtype=torch.float32, device=DEV)
    ops.tbe_backward(grad, w, None, None, _t(wo[:-1]), _t(do), _t(hs), _t(idx), _t(offs), T * D, D, 0, 3, 1.0,
                     total_hash_size_bits=int(hs[-1]).bit_length())
    delta = (w0 - w).view(-1, D)
    lin = np.concatenate([idx[t * B:(t + 1) * B] + hs[t] for t in range(T)])
    counts = np.bincount(lin, minlength=int(hs[-1])).astype(np.float32)
    # every element of a row moved by exactly its occurrence count (exact in fp32 for these magnitudes? no:
    # w - n is rounded; compare against the same fp32 computation)
    exp = w0.view(-1, D) + torch.as_tensor(counts, device=DEV)[:, None] * -1.0
    assert torch.equal(w.view(-1, D), exp)
    assert float(delta.sum().item()) == pytest.approx(float(T * B * D), rel=1e-3)
