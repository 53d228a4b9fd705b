"""Glue between torch tensors and the C ABI: enum codes, pointer extraction, status checks."""
import contextlib
import ctypes
import os

import torch

from ... import _clib

PT_BF16, PT_F16, PT_F32 = 0, 1, 2
PT_E4M3, PT_E5M2, PT_E2M1 = 0, 1, 2
PT_TENSORWISE, PT_ROWWISE, PT_BLOCKWISE, PT_MX_BLOCKWISE = 0, 1, 2, 3
PT_MX_ROW, PT_MX_COL, PT_MX_ROW_2D, PT_MX_COL_2D, PT_MX_ROW_RHT, PT_MX_COL_RHT = 1, 2, 4, 8, 16, 32
PT_MX_ROW_SR, PT_MX_COL_SR = 64, 128

_SRC = {torch.bfloat16: PT_BF16, torch.float16: PT_F16, torch.float32: PT_F32}
_FMT = {torch.float8_e4m3fn: PT_E4M3, torch.float8_e5m2: PT_E5M2, torch.float4_e2m1fn_x2: PT_E2M1}


check = _clib.check


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
_poll = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 the kernels write PT_ERR_TIMEOUT into if one of their bounded waits gives up.  The GEMM entry
    points get it as their `status` argument; it is also registered with the library as the word the quantizers (which
    have no such argument) report into."""
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        with torch.cuda.device(idx):
            check(lib().pt_set_default_status(ptr(_status[idx])), "set_default_status")
    return _status[idx]


def _raise(code):
    raise RuntimeError(f"a kernel gave up waiting on a barrier (status {code}); the output of that launch is invalid")


def check_status(device):
    """Synchronises and raises if a kernel reported an expired wait since the last check."""
    s = status_word(device)
    code = int(s.item())
    if code != 0:
        s.zero_()
        _raise(code)


def poll_status(device):
    """Called by the GEMM wrappers after a launch.  PT_CHECK_STATUS=1: a synchronising check_status().  Otherwise a check
    that never waits for the device: the status word is copied to pinned host memory asynchronously, at most one copy in
    flight; a later call that finds the copy complete reads it and raises if a kernel had given up.  An error therefore
    surfaces at a following operator call (or at an explicit check_status()), not at the launch that caused it."""
    if os.environ.get("PT_CHECK_STATUS") == "1":
        if not torch.cuda.is_current_stream_capturing():
            check_status(device)
        return
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    p = _poll.get(idx)
    if p is None:
        p = _poll[idx] = {"host": torch.zeros(1, dtype=torch.int32).pin_memory(), "event": None}
    if torch.cuda.is_current_stream_capturing():
        return
    ev = p["event"]
    if ev is not None:
        if not ev.query():
            return
        p["event"] = None
        code = int(p["host"][0])
        if code != 0:
            status_word(device).zero_()
            _raise(code)
    p["host"].copy_(status_word(device), non_blocking=True)
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(idx))
    p["event"] = ev


