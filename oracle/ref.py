"""TEST INFRASTRUCTURE ONLY: loaders for the reference's own compiled host code.

``oracle/_ref/libhybrid_cpp.so`` (``torch.classes.hybrid.IdsMapper``,
``torch.ops.hybrid.block_bucketize_sparse_features_cpu``) and
``oracle/_ref/libref_embcache.so`` (flat C ABI over ``Embcache::SwapManager``
and ``Embcache::FeatureFilter``) are produced by ``oracle/build_ref.py`` from
the reference tree.  ``available()`` tells whether they exist; nothing here
reads the reference tree at run time.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
HYBRID = os.path.join(HERE, "_ref", "libhybrid_cpp.so")
EMBCACHE = os.path.join(HERE, "_ref", "libref_embcache.so")

_hybrid_loaded = False
_emb = None
I64P = C.POINTER(C.c_int64)


def available() -> bool:
    return os.path.exists(HYBRID) and os.path.exists(EMBCACHE)


def load_hybrid():
    """Registers torch.classes.hybrid.IdsMapper / torch.ops.hybrid.*"""
    global _hybrid_loaded
    import torch

    if not _hybrid_loaded:
        torch.ops.load_library(HYBRID)
        _hybrid_loaded = True
    return torch


def embcache() -> C.CDLL:
    global _emb
    if _emb is None:
        import torch  # noqa: F401  (libtorch must be in the process before the harness)

        _emb = C.CDLL(EMBCACHE)
        _emb.ref_swap_new.restype = C.c_void_p
        _emb.ref_filter_new.restype = C.c_void_p
        for n in ("ref_swap_occupied", "ref_filter_num_evict", "ref_filter_count_of"):
            getattr(_emb, n).restype = C.c_int64
        _emb.ref_set_log_level(C.c_int(2))
    return _emb


def _p(a):
    return a.ctypes.data_as(I64P) if a is not None else None


class SwapManager:
    """The reference ``Embcache::SwapManager`` (swap_manager.h:28-55)."""

    def __init__(self, cache_size: int, mem_start_offset: int = 0):
        self._h = C.c_void_p(embcache().ref_swap_new(C.c_int64(cache_size), C.c_int64(mem_start_offset)))

    def __del__(self):
        if getattr(self, "_h", None):
            embcache().ref_swap_free(self._h)
            self._h = None

    def compute_swap_info(self, keys):
        keys = np.ascontiguousarray(keys, np.int64)
        n = keys.size
        m = max(n, 1)
        bo, sik, sio, sok, soo = (np.empty(m, np.int64) for _ in range(5))
        nin, nout = C.c_int64(0), C.c_int64(0)
        rc = embcache().ref_swap_compute(self._h, _p(keys), C.c_int64(n), _p(bo), _p(sik), _p(sio), C.byref(nin),
                                         _p(sok), _p(soo), C.byref(nout))
        if rc != 0:
            raise RuntimeError("cacheSize_ too small")
        return (sok[:nout.value].copy(), soo[:nout.value].copy(), sik[:nin.value].copy(), sio[:nin.value].copy(),
                bo[:n].copy())

    def remove_keys(self, keys):
        keys = np.ascontiguousarray(keys, np.int64)
        embcache().ref_swap_remove(self._h, _p(keys), C.c_int64(keys.size))

    def occupied(self) -> int:
        return embcache().ref_swap_occupied(self._h)


class FeatureFilter:
    """The reference ``Embcache::FeatureFilter`` (feature_filter.h:26-60)."""

    def __init__(self, admit_threshold: int = -1, evict_threshold: int = 0, evict_step_interval: int = 0):
        self._h = C.c_void_p(embcache().ref_filter_new(C.c_int64(admit_threshold), C.c_uint64(evict_threshold),
                                                       C.c_uint64(evict_step_interval)))

    def __del__(self):
        if getattr(self, "_h", None):
            embcache().ref_filter_free(self._h)
            self._h = None

    def statistics_key_count(self, keys, counts=None):
        keys = np.ascontiguousarray(keys, np.int64)
        counts = np.ascontiguousarray(counts, np.int64) if counts is not None else None
        embcache().ref_filter_statistics(self._h, _p(keys), _p(counts), C.c_int64(keys.size))

    def count_filter(self, keys):
        keys = np.ascontiguousarray(keys, np.int64).copy()
        embcache().ref_filter_count_filter(self._h, _p(keys), C.c_int64(keys.size))
        return keys

    def record_timestamp(self, keys, ts):
        keys = np.ascontiguousarray(keys, np.int64)
        ts = np.ascontiguousarray(ts, np.int64)
        embcache().ref_filter_record_timestamp(self._h, _p(keys), _p(ts), C.c_int64(keys.size))

    def evict_keys(self):
        n = embcache().ref_filter_num_evict(self._h)
        out = np.empty(max(n, 1), np.int64)
        embcache().ref_filter_get_evict(self._h, _p(out))
        return out[:n].copy()

    def clear_evict(self):
        embcache().ref_filter_clear_evict(self._h)

    def count_of(self, key: int) -> int:
        return embcache().ref_filter_count_of(self._h, C.c_int64(key))
