"""The pooled forward kernel's SIMT logic on the CPU: the kernel source itself (recsdk_b200/csrc/tbe_forward.cu) is
compiled with g++ against a host-side SIMT emulation (tests/emu/simt_emu.h: a std::thread per CUDA thread, warp
collectives as rendezvous points) and must reproduce the oracle bit for bit.  The emulation aborts when a warp
collective is reached by only part of its mask or with different operations -- undefined behaviour on a GPU that a
GPU run may or may not expose.  Small grids and blocks: every shuffle is a mutex round trip."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from oracle import port

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(HERE, "emu", "emu_forward.cpp")
OUT = os.path.join(HERE, "emu", "build", "libemu_forward.so")


@pytest.fixture(scope="module")
def emu():
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    deps = [SRC, os.path.join(HERE, "emu", "simt_emu.h"), os.path.join(ROOT, "recsdk_b200", "csrc", "tbe_forward.cu"),
            os.path.join(ROOT, "recsdk_b200", "csrc", "common.cuh"), os.path.join(ROOT, "include", "recsdk_b200.h")]
    if not os.path.exists(OUT) or any(os.path.getmtime(d) > os.path.getmtime(OUT) for d in deps):
        subprocess.check_call(["g++", "-O1", "-std=c++17", "-pthread", "-fPIC", "-shared", "-w",
                               f"-I{os.path.join(ROOT, 'include')}", f"-I{os.path.join(ROOT, 'recsdk_b200', 'csrc')}",
                               "-o", OUT, SRC])
    lib = C.CDLL(OUT)
    vp = C.c_void_p
    lib.emu_tbe_forward_pooled.restype = C.c_int
    lib.emu_tbe_forward_pooled.argtypes = [vp, vp, vp, vp, vp, vp, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32,
                                           C.c_int32, C.c_int64, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp,
                                           C.c_int64, C.c_int32, vp]
    return lib


def _case(rng, rows, dims, B, max_len, empty_frac):
    T = len(rows)
    wo = np.concatenate([[0], np.cumsum([r * d for r, d in zip(rows, dims)])]).astype(np.int64)
    do = np.concatenate([[0], np.cumsum(dims)]).astype(np.int32)
    lens = rng.integers(0 if empty_frac > 0 else 1, max_len + 1, size=T * B)
    lens[rng.random(T * B) < empty_frac] = 0
    idx = np.concatenate([rng.integers(0, rows[i // B], size=lens[i]) for i in range(T * B)] + [np.empty(0, np.int64)])
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    w = rng.uniform(-1, 1, int(wo[-1])).astype(np.float32)
    return dict(T=T, B=B, wo=wo[:-1].copy(), do=do, idx=idx.astype(np.int64), offs=offs, w=w, total_D=int(do[-1]),
                max_D=max(dims), dims=dims)


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


CASES = [
    # rows, dims, B, max_len, empty_frac, G, K, grid, block
    ([40, 30], [128, 128], 37, 3, 0.2, 32, 1, 2, 64),     # the benchmark's shape: a warp per 32 bags
    ([50], [128], 70, 1, 0.0, 32, 1, 1, 64),              # one id per bag, several groups per warp (pipeline rotates)
    ([20, 25, 9], [32, 16, 32], 21, 5, 0.3, 8, 1, 2, 64),  # sub-warp groups, mixed widths
    ([15], [8], 45, 4, 0.5, 2, 1, 3, 32),                 # 2-lane groups, many empty bags
    ([12], [256], 9, 6, 0.1, 32, 2, 2, 32),               # two vectors per lane
    ([10], [1024], 5, 3, 0.0, 32, 2, 1, 32),              # several column passes over the same ids
    ([9, 7], [6, 10], 11, 3, 0.2, 2, 1, 1, 32),           # widths that are not multiples of 4: scalar path
]


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("case", range(len(CASES)))
def test_emulated_forward_matches_oracle(emu, case, mode):
    rows, dims, B, max_len, ef, G, K, grid, block = CASES[case]
    rng = np.random.default_rng(700 + case)
    c = _case(rng, rows, dims, B, max_len, ef)
    exp = port.tbe_forward(c["w"], c["wo"], c["do"], c["idx"], c["offs"], c["T"], B, c["total_D"], c["max_D"], mode)
    out = np.full((B, c["total_D"]), -7.0, np.float32)
    status = np.zeros(4, np.int64)
    idx = c["idx"] if c["idx"].size else np.zeros(1, np.int64)
    rc = emu.emu_tbe_forward_pooled(_ptr(c["w"]), _ptr(c["wo"]), _ptr(c["do"]), _ptr(idx), _ptr(c["offs"]), _ptr(out),
                                    c["T"], B, c["idx"].size, c["total_D"], c["max_D"], mode, c["w"].size, _ptr(status),
                                    G, K, grid, block, 0, None, 0, 0, None)
    assert rc == 0 and status[0] == 0
    np.testing.assert_array_equal(out, exp)


def test_emulated_forward_into_sample_shards(emu):
    """Two shard buffers with their own row stride and column order (what a peer-mapped run hands the kernel)."""
    rows, dims, B, G, K = [40, 30], [128, 128], 24, 32, 1
    rng = np.random.default_rng(9)
    c = _case(rng, rows, dims, B, 2, 0.1)
    exp = port.tbe_forward(c["w"], c["wo"], c["do"], c["idx"], c["offs"], c["T"], B, c["total_D"], c["max_D"], 0)
    Bs, stride = B // 2, 260
    col = np.array([128, 0], np.int32)
    bufs = [np.full((Bs, stride), -7.0, np.float32) for _ in range(2)]
    ptrs = (C.c_void_p * 2)(bufs[0].ctypes.data, bufs[1].ctypes.data)
    status = np.zeros(4, np.int64)
    rc = emu.emu_tbe_forward_pooled(_ptr(c["w"]), _ptr(c["wo"]), _ptr(c["do"]), _ptr(c["idx"]), _ptr(c["offs"]), None,
                                    c["T"], B, c["idx"].size, c["total_D"], c["max_D"], 0, c["w"].size, _ptr(status),
                                    G, K, 1, 64, 2, C.cast(ptrs, C.c_void_p), Bs, stride, _ptr(col))
    assert rc == 0 and status[0] == 0
    for s in range(2):
        for t in range(2):
            np.testing.assert_array_equal(bufs[s][:, col[t]:col[t] + 128], exp[s * Bs:(s + 1) * Bs, t * 128:(t + 1) * 128])
        np.testing.assert_array_equal(bufs[s][:, 256:], np.full((Bs, 4), -7.0, np.float32))
