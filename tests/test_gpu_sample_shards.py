"""The sample-sharded output / gradient addressing of the forward and backward kernels, exercised on ONE GPU:
the shards are separate buffers on the same device with their own row stride and column order, exactly what
the peer-mapped buffers of a table-wise sharded run look like to the kernels.  Results must equal the oracle's
bit for bit after undoing the layout on the host."""
import numpy as np
import pytest
import torch

from oracle import port
from tests.test_gpu_tbe import DEV, _t, make_case

pytestmark = pytest.mark.gpu

CASES = [
    dict(rows=[200, 300, 120], dims=[8, 16, 8], B=32, max_len=6),
    dict(rows=[40, 8000], dims=[128, 128], B=300, max_len=3, alpha=1.3),
    dict(rows=[4000, 8000, 500], dims=[128, 128, 128], B=96, max_len=1, one_hot=True),
    dict(rows=[90, 60], dims=[6, 10], B=12, max_len=4),  # scalar path
]


def _layout(c, rng, pad):
    """Shard layout: features in a shuffled column order inside rows that are `pad` floats wider than needed."""
    T = c["T"]
    order = rng.permutation(T)
    col = np.zeros(T, np.int32)
    o = 0
    for t in order:
        col[t] = o
        o += c["dims"][t]
    return col, o + pad


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("case", range(len(CASES)))
def test_forward_into_sample_shards(case, mode, world):
    from recsdk_b200 import ops

    rng = np.random.default_rng(4000 + case)
    c = make_case(rng, **CASES[case])
    if c["B"] % world:
        pytest.skip("batch does not split evenly")
    Bs = c["B"] // world
    pad = 4 if all(d % 4 == 0 for d in c["dims"]) else 1
    col, stride = _layout(c, rng, pad)
    exp = port.tbe_forward(c["w"], c["wo"], c["do"], c["indices"], c["offsets"], c["T"], c["B"], c["total_D"],
                           c["max_D"], mode)
    bufs = [torch.full((Bs, stride), -7.0, dtype=torch.float32, device=DEV) for _ in range(world)]
    sh = ops.SampleShards([b.data_ptr() for b in bufs], Bs, stride, _t(col))
    st = ops.new_status(DEV)
    r = ops.tbe_forward(_t(c["w"]), _t(c["wo"]), _t(c["do"]), _t(c["indices"]), _t(c["offsets"]), c["total_D"],
                        c["max_D"], mode, status=st, out_shards=sh)
    assert r is None
    ops.raise_on_status(st)
    for s in range(world):
        got = bufs[s].cpu().numpy()
        for t in range(c["T"]):
            d0, d1 = c["do"][t], c["do"][t + 1]
            np.testing.assert_array_equal(got[:, col[t]:col[t] + (d1 - d0)], exp[s * Bs:(s + 1) * Bs, d0:d1])
        np.testing.assert_array_equal(got[:, stride - pad:], np.full((Bs, pad), -7.0, np.float32))  # padding untouched


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("opt", [1, 2, 3])
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("case", range(len(CASES)))
def test_backward_from_sample_shards(case, mode, opt, world):
    from recsdk_b200 import ops

    rng = np.random.default_rng(5000 + case)
    c = make_case(rng, **CASES[case])
    if c["B"] % world:
        pytest.skip("batch does not split evenly")
    Bs = c["B"] // world
    pad = 4 if all(d % 4 == 0 for d in c["dims"]) else 1
    col, stride = _layout(c, rng, pad)
    grad = rng.standard_normal((c["B"], c["total_D"])).astype(np.float32)
    shard_np = [np.zeros((Bs, stride), np.float32) for _ in range(world)]
    for s in range(world):
        for t in range(c["T"]):
            d0, d1 = c["do"][t], c["do"][t + 1]
            shard_np[s][:, col[t]:col[t] + (d1 - d0)] = grad[s * Bs:(s + 1) * Bs, d0:d1]
    bufs = [_t(a) for a in shard_np]
    sh = ops.SampleShards([b.data_ptr() for b in bufs], Bs, stride, _t(col))
    w = c["w"].copy()
    m1 = np.full_like(w, 0.1) if opt == 1 else rng.uniform(0, 0.01, w.size).astype(np.float32)
    m2 = rng.uniform(0, 0.01, w.size).astype(np.float32)
    dw, dm1, dm2 = _t(w), _t(m1), _t(m2)
    st = ops.new_status(DEV)
    bits = int(c["hs"][-1]).bit_length()
    for it in (1, 2):
        port.tbe_backward(grad, w, m1, m2, c["wo"], c["do"], c["hs"], c["indices"], c["offsets"], c["T"], c["B"],
                          c["total_D"], c["max_D"], mode, opt, 0.05, 1e-8, 0.9, 0.999, it, reduce_chunk=64)
        ops.tbe_backward(None, dw, dm1, dm2, _t(c["wo"]), _t(c["do"]), _t(c["hs"]), _t(c["indices"]),
                         _t(c["offsets"]), c["total_D"], c["max_D"], mode, opt, 0.05, 1e-8, 0.9, 0.999, it,
                         total_hash_size_bits=bits, reduce_chunk=64, status=st, grad_shards=sh)
    ops.raise_on_status(st)
    np.testing.assert_array_equal(dw.cpu().numpy(), w)
    if opt != 3:
        np.testing.assert_array_equal(dm1.cpu().numpy(), m1)
    if opt == 2:
        np.testing.assert_array_equal(dm2.cpu().numpy(), m2)


def test_sample_shards_reject_bad_descriptions():
    from recsdk_b200 import ops

    w = torch.zeros(64, dtype=torch.float32, device=DEV)
    buf = torch.zeros((2, 8), dtype=torch.float32, device=DEV)
    col = _t([0], torch.int32)
    # 2 shards x 2 samples != B = 3
    with pytest.raises(RuntimeError):
        ops.tbe_forward(w, _t([0]), _t([0, 8], torch.int32), _t([0, 1, 2]), _t([0, 1, 2, 3]), 8, 8, 0,
                        out_shards=ops.SampleShards([buf.data_ptr(), buf.data_ptr()], 2, 8, col))
    # NONE pooling has no sample-sharded form
    with pytest.raises(RuntimeError):
        ops.tbe_forward(w, _t([0]), _t([0, 8], torch.int32), _t([0, 1]), _t([0, 1, 2]), 8, 8, 2,
                        out_shards=ops.SampleShards([buf.data_ptr()], 2, 8, col))
