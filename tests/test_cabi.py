"""The C-ABI library loads and exports exactly what include/edm_b200.h declares.  No compute
calls here: only symbols, signatures and argument validation that returns before any launch."""
import ctypes as C
import os
import re

import pytest

from edmir_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "edm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(edm_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(native_lib):
    names = _declared()
    assert len(names) >= 20
    for name in names:
        assert hasattr(native_lib, name), f"{name} declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names
    assert native_lib.edm_version() == 1


def test_struct_layouts_match_header():
    assert C.sizeof(_lib.TpCall) == 128
    assert C.sizeof(_lib.CostParams) == 56
    assert C.sizeof(_lib.CandidateCost) == 40


def test_argument_validation_without_device(native_lib):
    # null pointers and bad extents are rejected before anything touches a device
    assert native_lib.edm_gemm_bf16(None, 8, None, 8, None, 8, 8, 8, 8, None) == _lib.EDM_ERR_BAD_ARG
    assert native_lib.edm_gemm_bf16(16, 8, 16, 8, 16, 8, 0, 8, 8, None) == _lib.EDM_ERR_BAD_ARG
    assert native_lib.edm_gemm_fp32_workspace_bytes(0, 1, 1) == 0
    assert native_lib.edm_gemm_fp32_workspace_bytes(256, 1024, 512) == 2 * 4 * (256 * 512 + 1024 * 512) + 256 * 128 * 256 * 4
    # extents whose byte counts would wrap around size_t are refused, not truncated
    assert native_lib.edm_gemm_fp32_workspace_bytes(1 << 30, 1 << 30, 1 << 30) == 0
    assert native_lib.edm_gemm_fp32_static(16, 1 << 30, 16, 1 << 30, 16, 1 << 30, 1 << 30, 1 << 30, 1 << 30,
                                           None) == _lib.EDM_ERR_CAPACITY
    assert native_lib.edm_gemm_fp32(16, 1 << 30, 16, 1 << 30, 16, 1 << 30, 1 << 30, 1 << 30, 1 << 30, 256, 1 << 40,
                                    None) == _lib.EDM_ERR_CAPACITY
    assert native_lib.edm_set_timeout_ms(0) == _lib.EDM_ERR_BAD_ARG
    out = C.c_void_p()
    assert native_lib.edm_comm_create(3, 2, 1 << 20, 1 << 20, C.byref(out)) == _lib.EDM_ERR_BAD_ARG
    assert native_lib.edm_comm_rank(None) == -1
    assert native_lib.edm_tp_launch(None, None, None) == _lib.EDM_ERR_BAD_ARG


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import pytest

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib._build, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_host_staging_needs_a_device():
    import torch
    from edmir_b200 import host_io
    if torch.cuda.is_available():
        pytest.skip("covered by the GPU suite")
    with pytest.raises(RuntimeError):
        host_io.HostStaging()
