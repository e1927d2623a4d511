"""The torch custom-op front (``TORCH_LIBRARY(b200_decode, ...)``): registration, schemas, loud failure on CPU.

No kernel runs here; the GPU suites exercise every operator through ``megatron_mixtera_b200.ops``.
"""
import pytest
import torch


@pytest.fixture(scope="module")
def b200_ops():
    from megatron_mixtera_b200 import _lib, build

    build.build_torch_ops()
    return _lib.load_torch_ops()


def test_every_operator_is_registered(b200_ops):
    from megatron_mixtera_b200 import _lib

    for name in _lib.TORCH_OPS:
        packet = getattr(b200_ops, name)
        schema = packet.default._schema
        assert schema.name == f"b200_decode::{name}"
        # outputs are caller-provided tensors marked as written; nothing is allocated behind the caller's back
        assert any(a.alias_info is not None and a.alias_info.is_write for a in schema.arguments), name
        assert len(schema.returns) == (1 if name == "gemm_splitk" else 0)


def test_ops_module_calls_the_torch_ops(b200_ops):
    """`ops.py` reaches the kernels through torch.ops only: its ctypes use is limited to calls that launch nothing."""
    import inspect
    import re

    from megatron_mixtera_b200 import ops

    src = inspect.getsource(ops)
    direct = set(re.findall(r"\.(b200_[a-z0-9_]+)\(", src))
    allowed_suffixes = ("_bytes", "_supported")
    allowed = {"b200_device_status", "b200_set_wait_limit_ns", "b200_copy_rows_h2d", "b200_fp8_value_position"}
    assert all(name in allowed or name.endswith(allowed_suffixes) for name in direct), direct


def test_cpu_tensors_are_refused(b200_ops):
    from megatron_mixtera_b200 import ops

    logits = torch.zeros(2, 8, dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        b200_ops.argmax(logits, torch.zeros(2, dtype=torch.int64))
    with pytest.raises(ops.B200Error):
        ops.argmax(logits)


def test_struct_blob_shares_memory():
    from megatron_mixtera_b200 import ops
    from megatron_mixtera_b200._lib import AttentionArgs
    import ctypes

    a = AttentionArgs()
    blob = ops._blob(a)
    assert blob.numel() == ctypes.sizeof(AttentionArgs) and blob.dtype == torch.uint8
    a.num_tokens = 77
    assert bytes(blob.numpy().tobytes()) == bytes(a)
    assert ops._blob(a) is blob
