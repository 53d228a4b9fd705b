"""The C-ABI library loads on a machine without a GPU and exports every function include/pt_b200.h declares;
the ctypes table mirrors the header one to one.  No compute call is made here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "pt_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pt_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_functions():
    names = declared_functions()
    assert "pt_gemm_fp8" in names and "pt_quantize_mx" in names and len(names) >= 15


def test_library_exports_every_declared_symbol():
    from primus_turbo import _clib
    lib = ctypes.CDLL(_clib.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in pt_b200.h but not exported by libpt_b200.so"


def test_ctypes_table_matches_header():
    from primus_turbo import _clib
    assert sorted(_clib.SIGNATURES) == declared_functions()
    text = open(os.path.join(ROOT, "include", "pt_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    for name, (_, args) in _clib.SIGNATURES.items():
        m = re.search(r"\b" + name + r"\s*\(([^;]*?)\)\s*;", text, flags=re.S)
        assert m, name
        params = [p for p in m.group(1).split(",") if p.strip() and p.strip() != "void"]
        assert len(params) == len(args), f"{name}: header has {len(params)} parameters, ctypes table {len(args)}"


def test_errors_without_gpu_are_reported_not_hidden():
    """Argument validation happens before any CUDA call, so it can be exercised on a CPU-only box."""
    from primus_turbo import _clib
    lib = _clib.load()
    rc = lib.pt_quantize_mx(None, 0, 1, 64, 48, 0, 1, None, None, None, None, None)
    assert rc == -1 and b"divisible by 32" in lib.pt_last_error()
    rc = lib.pt_gemm_fp8(None, None, 0, None, None, 0, None, 0, 0, 128, 128, 100, 0.0, 0, None, 0, None, None)
    assert rc == -1 and b"multiple of 16" in lib.pt_last_error()
    with pytest.raises(RuntimeError, match="failed"):
        _clib.check(rc, "pt_gemm_fp8")


def test_ops_refuse_cpu_tensors():
    import torch
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        qi.quantize_fp8_tensorwise_impl(torch.zeros(4, 4), torch.float8_e4m3fn)
