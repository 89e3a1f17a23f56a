"""The torch custom ops are registered with exactly the reference's schemas (fixture: tests/golden/op_schemas.txt,
extracted from the reference's registration by tests/golden/make_schemas.py)."""
import os

import pytest
import torch


def test_registered_schemas_equal_reference(golden_dir):
    from recsdk_b200 import torch_ops

    if not torch_ops.available():
        pytest.skip("torch op library not built")
    torch_ops.load()
    want = [l.strip() for l in open(os.path.join(golden_dir, "op_schemas.txt")) if l.strip()]
    assert len(want) == 7
    for schema in want:
        name = schema.split("(")[0]
        for ns in ("fbgemm", "recsdk"):
            op = getattr(getattr(torch.ops, ns), name).default
            got = str(op._schema).replace(f"{ns}::", "", 1)
            assert got == schema, f"{ns}::{name}"


def test_ids_mapper_class_and_bucketize_are_registered():
    from recsdk_b200 import torch_ops

    if not torch_ops.available():
        pytest.skip("torch op library not built")
    torch_ops.load()
    assert torch.classes.recsdk.IdsMapper is not None
    s = str(torch.ops.recsdk.block_bucketize_sparse_features.default._schema)
    assert s.count("Tensor") >= 10 and "bool" in s
    # the reference's own names (hybrid_torchrec/src/bind_torch_lib.cpp:9-19)
    assert torch.classes.hybrid.IdsMapper is not None
    assert str(torch.ops.hybrid.block_bucketize_sparse_features_cpu.default._schema).count("Tensor") >= 10
