"""Glue between torch tensors and the C ABI: enum codes, pointer extraction, status checks."""
import contextlib
import ctypes

import torch

from ... import _clib

PT_BF16, PT_F16, PT_F32 = 0, 1, 2
PT_E4M3, PT_E5M2, PT_E2M1 = 0, 1, 2
PT_TENSORWISE, PT_ROWWISE, PT_BLOCKWISE, PT_MX_BLOCKWISE = 0, 1, 2, 3
PT_MX_ROW, PT_MX_COL, PT_MX_ROW_2D, PT_MX_COL_2D, PT_MX_ROW_RHT, PT_MX_COL_RHT = 1, 2, 4, 8, 16, 32

_SRC = {torch.bfloat16: PT_BF16, torch.float16: PT_F16, torch.float32: PT_F32}
_FMT = {torch.float8_e4m3fn: PT_E4M3, torch.float8_e5m2: PT_E5M2, torch.float4_e2m1fn_x2: PT_E2M1}


def lib():
    return _clib.load()


def src_code(dtype) -> int:
    try:
        return _SRC[dtype]
    except KeyError:
        raise TypeError(f"unsupported high-precision dtype {dtype}") from None


def fmt_code(dtype) -> int:
    try:
        return _FMT[dtype]
    except KeyError:
        raise TypeError(f"unsupported quantized dtype {dtype}") from None


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream(device=None):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


_NO_GUARD = contextlib.nullcontext()


def on_device(device):
    """Context in which `device` is the current CUDA device; free when it already is (the usual case: one process
    per GPU), a torch device guard otherwise."""
    idx = device.index
    if idx is None or idx == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("primus_turbo (B200) operators take CUDA tensors only; there is no CPU path")


_status = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 the GEMM kernels write PT_ERR_TIMEOUT into if one of their bounded waits expires."""
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
    return _status[idx]


def check_status(device):
    """Synchronises and raises if a kernel reported an expired wait (debug / test helper)."""
    s = status_word(device)
    code = int(s.item())
    if code != 0:
        s.zero_()
        raise RuntimeError(f"a GEMM kernel gave up waiting on a barrier (status {code}); its output is invalid")


check = _clib.check
