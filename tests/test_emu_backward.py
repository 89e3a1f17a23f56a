"""The backward kernels' SIMT logic on the CPU (expand -> [host sort] -> per-run records -> partial sums -> row
update), compiled from the kernel source itself against tests/emu/simt_emu.h, against the oracle bit for bit.
See test_emu_forward.py for what the emulation checks beyond the numbers."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from oracle import port

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(HERE, "emu", "emu_backward.cpp")
OUT = os.path.join(HERE, "emu", "build", "libemu_backward.so")


@pytest.fixture(scope="module")
def emu():
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    deps = [SRC, os.path.join(HERE, "emu", "simt_emu.h"), os.path.join(ROOT, "recsdk_b200", "csrc", "tbe_backward.cuh"),
            os.path.join(ROOT, "recsdk_b200", "csrc", "common.cuh"), os.path.join(ROOT, "include", "recsdk_b200.h")]
    if not os.path.exists(OUT) or any(os.path.getmtime(d) > os.path.getmtime(OUT) for d in deps):
        subprocess.check_call(["g++", "-O1", "-std=c++17", "-pthread", "-fPIC", "-shared", "-w", "-ffp-contract=off",
                               f"-I{os.path.join(ROOT, 'include')}", f"-I{os.path.join(ROOT, 'recsdk_b200', 'csrc')}",
                               "-o", OUT, SRC])
    lib = C.CDLL(OUT)
    vp = C.c_void_p
    lib.emu_tbe_backward.restype = C.c_int
    lib.emu_tbe_backward.argtypes = [vp] * 9 + [C.c_int64] * 3 + [C.c_int32] * 5 + [C.c_float] * 5 + [C.c_int64, vp] + \
        [C.c_int] * 4
    return lib


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


CASES = [
    # rows, dims, B, max_len, hot (ids drawn from the first `hot` rows every 3rd bag), G, K, grid, block
    ([40, 30], [128, 128], 37, 3, 5, 32, 1, 2, 64),
    ([6], [128], 150, 1, 2, 32, 1, 2, 64),        # runs longer than 64: chunk sums
    ([20, 25, 9], [32, 32, 32], 21, 5, 3, 8, 1, 2, 64),
    ([15], [8], 45, 4, 4, 2, 1, 3, 32),
    ([12], [256], 9, 6, 2, 32, 2, 1, 32),
]


@pytest.mark.parametrize("opt", [1, 2, 3])
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("case", range(len(CASES)))
def test_emulated_backward_matches_oracle(emu, case, mode, opt):
    rows, dims, B, max_len, hot, G, K, grid, block = CASES[case]
    rng = np.random.default_rng(800 + case)
    T = len(rows)
    wo = np.concatenate([[0], np.cumsum([r * d for r, d in zip(rows, dims)])]).astype(np.int64)
    do = np.concatenate([[0], np.cumsum(dims)]).astype(np.int32)
    hs = np.concatenate([[0], np.cumsum(rows)]).astype(np.int64)
    lens = rng.integers(0 if max_len > 1 else 1, max_len + 1, size=T * B)
    idx = np.concatenate([rng.integers(0, hot if i % 3 == 0 else rows[i // B], size=lens[i]) for i in range(T * B)])
    idx = idx.astype(np.int64)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    total_D, max_D = int(do[-1]), max(dims)
    grad = rng.standard_normal((B, total_D)).astype(np.float32)
    w = rng.uniform(-1, 1, int(wo[-1])).astype(np.float32)
    m1 = np.full_like(w, 0.1) if opt == 1 else rng.uniform(0, 0.01, w.size).astype(np.float32)
    m2 = rng.uniform(0, 0.01, w.size).astype(np.float32)
    ew, em1, em2 = w.copy(), m1.copy(), m2.copy()
    status = np.zeros(4, np.int64)
    for it in (1, 2):
        port.tbe_backward(grad, ew, em1, em2, wo[:-1].copy(), do, hs, idx, offs, T, B, total_D, max_D, mode, opt, 0.05,
                          1e-8, 0.9, 0.999, it, reduce_chunk=64)
        b2s = port.adam_beta2sqrt(0.9, 0.999, it) if opt == 2 else 0.0
        wofs = wo[:-1].copy()
        rc = emu.emu_tbe_backward(_ptr(grad), _ptr(w), _ptr(m1), _ptr(m2), _ptr(wofs), _ptr(do), _ptr(hs), _ptr(idx),
                                  _ptr(offs), T, B, idx.size, total_D, max_D, mode, opt, 64, 0.05, 1e-8, 0.9, 0.999,
                                  b2s, w.size, _ptr(status), G, K, grid, block)
        assert rc == 0 and status[0] == 0
    np.testing.assert_array_equal(w, ew)
    if opt != 3:
        np.testing.assert_array_equal(m1, em1)
    if opt == 2:
        np.testing.assert_array_equal(m2, em2)


@pytest.mark.parametrize("opt", [1, 2, 3])
def test_emulated_backward_shared_table_unaligned_columns(emu, opt):
    """Features [A, B, A, C] with dims 8, 6, 8, 2: table A's rows could be moved 128 bits at a time, but feature 2's
    gradient columns start at 14, and a run of table A holds gradient rows of features 0 AND 2.  The kernels must
    fall back to the scalar path for every run (a float4 load at column 14 is misaligned on the GPU)."""
    rng = np.random.default_rng(77)
    rows, dims, ftm, B = [30, 20, 10], [8, 6, 2], [0, 1, 0, 2], 19
    T = len(ftm)
    table_wo = np.concatenate([[0], np.cumsum([r * d for r, d in zip(rows, dims)])]).astype(np.int64)
    table_hs = np.concatenate([[0], np.cumsum(rows)]).astype(np.int64)
    wo = np.array([table_wo[t] for t in ftm], np.int64)
    fd = [dims[t] for t in ftm]
    do = np.concatenate([[0], np.cumsum(fd)]).astype(np.int32)
    hs = np.array([table_hs[t] for t in ftm] + [table_hs[-1]], np.int64)
    lens = rng.integers(0, 4, size=T * B)
    idx = np.concatenate([rng.integers(0, min(6, rows[ftm[i // B]]), size=lens[i]) for i in range(T * B)]).astype(np.int64)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    total_D, max_D = int(do[-1]), max(fd)
    grad = rng.standard_normal((B, total_D)).astype(np.float32)
    w = rng.uniform(-1, 1, int(table_wo[-1])).astype(np.float32)
    m1 = np.full_like(w, 0.1)
    m2 = rng.uniform(0, 0.01, w.size).astype(np.float32)
    ew, em1, em2 = w.copy(), m1.copy(), m2.copy()
    status = np.zeros(4, np.int64)
    port.tbe_backward(grad, ew, em1, em2, wo.copy(), do, hs, idx, offs, T, B, total_D, max_D, 0, opt, 0.05, 1e-8, 0.9,
                      0.999, 1, reduce_chunk=64)
    b2s = port.adam_beta2sqrt(0.9, 0.999, 1) if opt == 2 else 0.0
    rc = emu.emu_tbe_backward(_ptr(grad), _ptr(w), _ptr(m1), _ptr(m2), _ptr(wo), _ptr(do), _ptr(hs), _ptr(idx),
                              _ptr(offs), T, B, idx.size, total_D, max_D, 0, opt, 64, 0.05, 1e-8, 0.9, 0.999, b2s,
                              w.size, _ptr(status), 2, 1, 2, 64)
    assert rc == 0 and status[0] == 0
    np.testing.assert_array_equal(w, ew)
    if opt != 3:
        np.testing.assert_array_equal(m1, em1)
    if opt == 2:
        np.testing.assert_array_equal(m2, em2)
