"""The C-ABI shared library: it builds, loads, and exports exactly what include/b200_decode.h declares.
No compute entry point is called here (this file runs without a GPU)."""
import ctypes
import os
import re

from conftest import ROOT


def header_functions():
    text = open(os.path.join(ROOT, "include", "b200_decode.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)  # comments mention symbols that are not declarations
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from megatron_mixtera_b200 import _lib, build

    path = build.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    declared = header_functions()
    assert len(declared) >= 40
    missing = [name for name in declared if not hasattr(lib, name)]
    assert not missing, missing
    # the typed loader knows the same set: no entry point without ctypes signatures, none undeclared
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared
    typed = _lib.load()
    for name in declared:
        assert getattr(typed, name).restype is not None or name == "b200_version"


def test_host_only_entry_points():
    from megatron_mixtera_b200 import _lib

    lib = _lib.load()
    assert lib.b200_version() >= 1
    assert lib.b200_error_string(0) and b"scratch" in lib.b200_error_string(-7)
    assert lib.b200_error_string(-12345)  # unknown codes still give a string
    assert lib.b200_gemm_bf16_static_scratch_limit() == 16 * 1024 * 1024
    assert lib.b200_mxfp8_scale_bytes(64, 4096) == 2 * 32 * 512 and lib.b200_mxfp8_scale_bytes(64, 100) == 0
    # FP8 value-pool positions: a permutation inside every 32 tokens
    pos = [lib.b200_fp8_value_position(t) for t in range(256)]
    assert sorted(pos) == list(range(256))
    assert all(p // 32 == t // 32 for t, p in enumerate(pos))
    # argument checks run before any CUDA call
    assert lib.b200_gemm_bf16(None, 0, None, None, None, 0, 0, 0, 0, None, 0, None) < 0
    assert lib.b200_paged_attention(None, None) < 0
    assert lib.b200_argmax_bf16(None, 0, None, 0, 0, None) < 0
