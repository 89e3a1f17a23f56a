"""The allocation-free dedup entry point (recsdk_unique_sorted_static) against the regular one.

Who needs it: code that may not allocate device memory when the dedup is due -- allocator callbacks and
memory-pool hooks, worker threads that were handed device buffers but no allocator, services with a fixed
device-memory budget.  The sort scratch is a __device__ array inside the library (limit
RECSDK_UNIQUE_STATIC_MAX_N ids), shared by every call on the device, so this test also runs it twice in a row:
the second call must not be disturbed by what the first one left behind.

This file sorts last on purpose (a run that stops at the first failure has then run everything else), and it
passes both on its own in a fresh process and after the rest of the suite.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _call_static(lib, ids, bits):
    n = ids.numel()
    uq = torch.full((max(n, 1),), -1, dtype=torch.int64, device=DEV)
    inv = torch.full((max(n, 1),), -1, dtype=torch.int64, device=DEV)
    cnt = torch.full((1,), -1, dtype=torch.int64, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    # warm-up: the first call on a device locates the array (and is when the driver loads this code's device image);
    # the check below is about the calls after it
    warm = torch.empty(0, dtype=torch.int64, device=DEV)
    assert lib.recsdk_unique_sorted_static(warm.data_ptr(), 0, 64, uq.data_ptr(), inv.data_ptr(), cnt.data_ptr(), st) == 0
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]
    rc = lib.recsdk_unique_sorted_static(ids.data_ptr(), n, bits, uq.data_ptr(), inv.data_ptr(), cnt.data_ptr(), st)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before  # nothing was allocated through torch
    assert torch.cuda.mem_get_info()[0] >= free_before  # nor by the driver: the device's free memory did not shrink
    return rc, uq, inv, cnt


def test_static_entry_point_matches_regular_entry_point_twice():
    from recsdk_b200 import _lib, ops

    lib = _lib.load()
    max_n = lib.recsdk_unique_sorted_static_max_n()
    assert max_n == 262144
    rng = np.random.default_rng(77)
    # two different inputs back to back on the same (shared) scratch: the full size, then a small one
    cases = [(max_n, 64, 2**62), (5000, 20, 2**20), (max_n, 33, 2**33)]
    for n, bits, vocab in cases:
        ids_np = rng.integers(0, vocab, size=n, dtype=np.int64)
        ids_np[: n // 2] = ids_np[n // 2: n // 2 * 2]  # plenty of duplicates
        ids = torch.from_numpy(ids_np).to(DEV)
        ref_uq, ref_inv, ref_cnt = ops.unique_sorted(ids, key_bits=bits)
        for _ in range(2):  # two calls in a row
            rc, uq, inv, cnt = _call_static(lib, ids, bits)
            assert rc == 0
            u = int(cnt.item())
            assert u == int(ref_cnt.item())
            assert torch.equal(uq[:u], ref_uq[:u])  # integer work: bit-exact
            assert torch.equal(inv[:n], ref_inv)


def test_static_entry_point_rejects_sizes_beyond_its_scratch():
    from recsdk_b200 import _lib

    lib = _lib.load()
    max_n = lib.recsdk_unique_sorted_static_max_n()
    ids = torch.zeros(max_n + 1, dtype=torch.int64, device=DEV)
    rc, _, _, _ = _call_static(lib, ids, 64)
    assert rc == _lib.ERR_TOO_LARGE
    assert "maximum" in _lib.error_string(rc)
    # empty input is fine and reports zero uniques
    rc, _, _, cnt = _call_static(lib, torch.empty(0, dtype=torch.int64, device=DEV), 64)
    assert rc == 0 and int(cnt.item()) == 0
