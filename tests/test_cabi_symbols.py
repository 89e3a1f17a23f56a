"""The C-ABI library loads and exports every symbol include/recsdk_b200.h declares (no compute calls)."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "recsdk_b200.h")).read()
    return sorted(set(re.findall(r"RECSDK_API\s+[\w\s\*]+?\b(recsdk_\w+)\s*\(", text)))


def test_header_declares_symbols():
    syms = _declared_symbols()
    assert len(syms) >= 30
    assert "recsdk_tbe_forward" in syms and "recsdk_tbe_backward" in syms


def test_library_exports_every_declared_symbol():
    from recsdk_b200 import _lib

    lib = _lib.load()
    declared = _declared_symbols()
    for s in declared:
        assert hasattr(lib, s), f"missing export {s}"
    # and the python binding table covers exactly the header
    assert sorted(_lib.SIGNATURES) == declared


def test_host_only_entry_points():
    from recsdk_b200 import _lib
    from oracle import port

    lib = _lib.load()
    assert lib.recsdk_version() >= 100
    assert _lib.error_string(_lib.ERR_CACHE_TOO_SMALL) == "cacheSize_ too small"
    for it in (1, 2, 10, 1000):
        assert lib.recsdk_adam_beta2sqrt(0.9, 0.999, it) == pytest.approx(port.adam_beta2sqrt(0.9, 0.999, it), abs=0)
    assert lib.recsdk_tbe_backward_workspace_bytes(1 << 20, 128) > (1 << 20) * 24
    # argument validation happens before any CUDA call
    assert lib.recsdk_tbe_forward(None, None) == _lib.ERR_INVALID_ARG
    assert lib.recsdk_unique_sorted(None, -1, 64, None, None, None, None, 0, None) == _lib.ERR_INVALID_ARG


def test_cpu_tensors_are_rejected():
    import torch
    from recsdk_b200 import ops

    w = torch.zeros(16)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ops.tbe_forward(w, torch.zeros(1, dtype=torch.int64), torch.tensor([0, 4], dtype=torch.int32),
                        torch.zeros(2, dtype=torch.int64), torch.tensor([0, 1, 2]), 4, 4, 0)
