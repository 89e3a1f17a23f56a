"""Loads the torch custom-op library (csrc_torch/torch_ops.cpp): `torch.ops.fbgemm.split_embedding_*` with the
reference's schemas, the same ops under `torch.ops.recsdk.*`, `torch.classes.recsdk.IdsMapper` and
`torch.ops.recsdk.block_bucketize_sparse_features`."""
from __future__ import annotations

import os

import torch

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "librecsdk_b200_torch.so")
_loaded = False


def available() -> bool:
    return os.path.exists(LIB_PATH)


def load() -> None:
    """Raises if the library was not built (`python -m recsdk_b200.build --torch`)."""
    global _loaded
    if _loaded:
        return
    if not available():
        raise ImportError(f"{LIB_PATH} not found: build it with `python -m recsdk_b200.build --torch`")
    from . import _lib

    _lib.load()  # librecsdk_b200.so first: the op library links against it
    torch.ops.load_library(LIB_PATH)
    _loaded = True


def is_loaded() -> bool:
    return _loaded
