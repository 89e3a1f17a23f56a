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


def test_kjt_utilities_are_registered():
    """cust_op/framework/torch_plugin/torch_library/2.6.0/{permute2d_sparse_data,permute1d_sparse_data,
    asynchronous_complete_cumsum,jagged_to_padded_dense,dense_to_jagged}: schema strings of their m.def calls."""
    from recsdk_b200 import torch_ops

    if not torch_ops.available():
        pytest.skip("torch op library not built")
    torch_ops.load()
    want = {
        "permute_2D_sparse_data": "(Tensor permute, Tensor lengths, Tensor values, Tensor? weights=None, "
                                  "SymInt? permuted_lengths_sum=None) -> (Tensor, Tensor, Tensor?)",
        "permute_1D_sparse_data": "(Tensor permute, Tensor lengths, Tensor values, Tensor? weights=None, "
                                  "SymInt? permuted_lengths_sum=None) -> (Tensor, Tensor, Tensor?)",
        "asynchronous_complete_cumsum": "(Tensor offset) -> Tensor",
        "dense_to_jagged": "(Tensor dense, Tensor[] offsets, SymInt? total_L=None) -> (Tensor, Tensor[])",
    }
    for ns in ("fbgemm", "mxrec", "recsdk"):
        for name, sig in want.items():
            got = [str(x) for x in torch._C._jit_get_schemas_for_operator(f"{ns}::{name}")]
            assert got == [f"{ns}::{name}{sig}"], (ns, name, got)
        got = sorted(str(x) for x in torch._C._jit_get_schemas_for_operator(f"{ns}::jagged_to_padded_dense"))
        assert got == [f"{ns}::jagged_to_padded_dense.v1(Tensor values, Tensor[] offsets, int max_lengths, "
                       "float padding_value) -> Tensor",
                       f"{ns}::jagged_to_padded_dense.v2(Tensor values, Tensor[] offsets, int[] max_lengths, "
                       "float padding_value) -> Tensor"]


def test_tf_flavour_operators_are_registered():
    """cust_op/framework/tf_plugin/src/{cust_embedding_by_address,lazy_adam,sgd}.cpp: same operator names, input order
    and attribute names as the REGISTER_OP blocks."""
    from recsdk_b200 import torch_ops

    if not torch_ops.available():
        pytest.skip("torch op library not built")
    torch_ops.load()
    want = {
        "EmbeddingLookupByAddress": ["address", "embedding_dim", "embedding_type"],
        "EmbeddingUpdateByAddress": ["address", "embedding", "update_type"],
        "LazyAdam": ["gradient", "indices", "input_m", "input_v", "input_var", "lr", "beta1", "beta2", "epsilon"],
        "Sgd": ["gradient", "indices", "input_var", "lr", "weightDecay"],
    }
    for name, args in want.items():
        schema = getattr(torch.ops.recsdk, name).default._schema
        assert [a.name for a in schema.arguments] == args
