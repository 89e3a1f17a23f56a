"""Jagged-batch utilities (permute_2D / permute_1D sparse data, complete cumsum, jagged <-> padded dense) through
the C ABI against the numpy restatement, bit for bit (pure data movement and integer sums); shapes and dtype
combinations follow the reference operator tests
(cust_op/test/{permute2d_sparse_data,permute1d_sparse_data,asynchronous_complete_cumsum,jagged_to_padded_dense}_test)."""
import numpy as np
import pytest
import torch

from oracle import port

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.mark.parametrize("ltype", [np.int64, np.int32])
@pytest.mark.parametrize("vtype", [np.int64, np.int32, np.float32])
@pytest.mark.parametrize("with_w", [False, True])
@pytest.mark.parametrize("shape", [(5, 0, 64), (7, 3, 2048), (12, -4, 333), (3, 2, 20480)])
@pytest.mark.parametrize("give_sum", [True, False])
def test_permute_2d_sparse_data(ltype, vtype, with_w, shape, give_sum):
    from recsdk_b200 import ops

    t, extra, B = shape
    rng = np.random.default_rng(abs(hash((t, extra, B))) % 2**31)
    T_in = t + extra
    permute = rng.choice(T_in, t).astype(np.int32)
    lengths = rng.integers(0, 4, size=(T_in, B)).astype(ltype)
    n = int(lengths.sum())
    values = (rng.integers(0, 10**6, n) if vtype != np.float32 else rng.standard_normal(n)).astype(vtype)
    weights = rng.standard_normal(n).astype(np.float32) if with_w else None
    el, ev, ew = port.permute_2D_sparse_data(permute, lengths, values, weights)
    gl, gv, gw = ops.permute_2D_sparse_data(_t(permute), _t(lengths), _t(values), _t(weights) if with_w else None,
                                            int(el.sum()) if give_sum else None)
    assert gl.dtype == _t(lengths).dtype and gv.dtype == _t(values).dtype
    np.testing.assert_array_equal(gl.cpu().numpy(), el)
    np.testing.assert_array_equal(gv.cpu().numpy(), ev)
    if with_w:
        np.testing.assert_array_equal(gw.cpu().numpy(), ew)
    else:
        assert gw is None


def test_permute_1d_sparse_data_and_errors():
    from recsdk_b200 import ops

    rng = np.random.default_rng(3)
    lengths = rng.integers(0, 6, 500).astype(np.int64)
    values = rng.integers(0, 1000, int(lengths.sum())).astype(np.int64)
    permute = rng.permutation(500)[:300].astype(np.int32)
    el, ev, _ = port.permute_1D_sparse_data(permute, lengths, values)
    gl, gv, gw = ops.permute_1D_sparse_data(_t(permute), _t(lengths), _t(values))
    np.testing.assert_array_equal(gl.cpu().numpy(), el)
    np.testing.assert_array_equal(gv.cpu().numpy(), ev)
    assert gw is None
    with pytest.raises(RuntimeError, match="out of range"):
        ops.permute_1D_sparse_data(_t(np.array([0, 700], np.int32)), _t(lengths), _t(values), None, 10)
    with pytest.raises(RuntimeError, match="weights and values length mismatch"):
        ops.permute_1D_sparse_data(_t(permute), _t(lengths), _t(values), _t(np.zeros(3, np.float32)))


@pytest.mark.parametrize("n", [1, 7, 2048, 2049, 100000, 1703936])
@pytest.mark.parametrize("dtype", [np.int64, np.int32])
def test_asynchronous_complete_cumsum(n, dtype):
    from recsdk_b200 import ops

    x = np.random.default_rng(n).integers(0, 100, n).astype(dtype)
    got = ops.asynchronous_complete_cumsum(_t(x))
    assert got.dtype == _t(x).dtype
    np.testing.assert_array_equal(got.cpu().numpy(), port.asynchronous_complete_cumsum(x))


@pytest.mark.parametrize("D", [1, 6, 32, 128])
@pytest.mark.parametrize("B,max_len,L", [(1, 5, 5), (37, 9, 6), (400, 20, 30)])
def test_jagged_dense_round_trip(D, B, max_len, L):
    """L < max_len truncates rows (their jagged gradient is zero), L > max_len pads."""
    from recsdk_b200 import ops

    rng = np.random.default_rng(D * 1000 + B)
    lens = rng.integers(0, max_len + 1, B)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    values = rng.standard_normal((int(offs[-1]), D)).astype(np.float32)
    exp = port.jagged_to_padded_dense(values, offs, L, -1.5)
    got = ops.jagged_to_padded_dense(_t(values), [_t(offs)], L, -1.5)
    np.testing.assert_array_equal(got.cpu().numpy(), exp)
    got2 = ops.jagged_to_padded_dense(_t(values), [_t(offs)], [L], -1.5)  # the int[] form
    np.testing.assert_array_equal(got2.cpu().numpy(), exp)
    dense = rng.standard_normal((B, L, D)).astype(np.float32)
    back, _ = ops.dense_to_jagged(_t(dense), [_t(offs)])
    np.testing.assert_array_equal(back.cpu().numpy(), port.dense_to_jagged(dense, offs))
    with pytest.raises(RuntimeError, match="max_lengths must be positive"):
        ops.jagged_to_padded_dense(_t(values), [_t(offs)], 0, 0.0)
    with pytest.raises(RuntimeError, match="exactly 1 tensor"):
        ops.jagged_to_padded_dense(_t(values), [_t(offs), _t(offs)], L, 0.0)


@pytest.mark.parametrize("ns", ["fbgemm", "mxrec", "recsdk"])
def test_registered_kjt_ops(ns):
    """The operators under the names the reference registers them with (mxrec:: definitions, fbgemm:: callers)."""
    from recsdk_b200 import torch_ops

    if not torch_ops.available():
        pytest.skip("torch op library not built")
    torch_ops.load()
    o = getattr(torch.ops, ns)
    rng = np.random.default_rng(1)
    lengths = rng.integers(0, 4, size=(6, 50)).astype(np.int64)
    values = rng.integers(0, 999, int(lengths.sum())).astype(np.int64)
    permute = np.array([3, 0, 5, 3], np.int32)
    el, ev, _ = port.permute_2D_sparse_data(permute, lengths, values)
    gl, gv, gw = o.permute_2D_sparse_data(_t(permute), _t(lengths), _t(values))
    np.testing.assert_array_equal(gl.cpu().numpy(), el)
    np.testing.assert_array_equal(gv.cpu().numpy(), ev)
    assert gw is None
    l1 = lengths.reshape(-1)
    p1 = rng.permutation(l1.size).astype(np.int32)
    el, ev, _ = port.permute_1D_sparse_data(p1, l1, values)
    gl, gv, _ = o.permute_1D_sparse_data(_t(p1), _t(l1), _t(values), None, int(el.sum()))
    np.testing.assert_array_equal(gl.cpu().numpy(), el)
    np.testing.assert_array_equal(gv.cpu().numpy(), ev)
    np.testing.assert_array_equal(o.asynchronous_complete_cumsum(_t(l1)).cpu().numpy(),
                                  port.asynchronous_complete_cumsum(l1))
    # jagged <-> dense with autograd: the gradient of the padded tensor flows back to the jagged rows
    offs = np.concatenate([[0], np.cumsum(rng.integers(0, 7, 20))]).astype(np.int64)
    vals = torch.randn(int(offs[-1]), 16, device=DEV, requires_grad=True)
    dense = o.jagged_to_padded_dense(vals, [_t(offs)], 5, 0.0)
    np.testing.assert_array_equal(dense.detach().cpu().numpy(),
                                  port.jagged_to_padded_dense(vals.detach().cpu().numpy(), offs, 5, 0.0))
    g = torch.randn_like(dense)
    dense.backward(g)
    np.testing.assert_array_equal(vals.grad.cpu().numpy(), port.dense_to_jagged(g.cpu().numpy(), offs))
    jag, out_offs = o.dense_to_jagged(g, [_t(offs)], int(offs[-1]))
    np.testing.assert_array_equal(jag.cpu().numpy(), port.dense_to_jagged(g.cpu().numpy(), offs))
    assert len(out_offs) == 1
